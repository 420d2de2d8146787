"""Record what the REFERENCE's own ``cuBladeW8A16LinearLayer`` computes on a B200 (run on a GPU box).

The reference package, installed unmodified into ``oracle/_ref/site`` by ``oracle/build_ref.py``, is
imported as ``cublade``; its layer (``cublade/quantization/linear.py:8-137``) is built on the seeded
inputs of ``tests/golden/cases.py`` -- the benchmark shape N = 14336, K = 4096 at M in {1, 16, 128,
2048}, once plain and once as the LLM.int8 variant with 8 outlier columns and a bias -- and its own
``quantize()`` and ``forward()`` run: the reference's CUDA per-channel quantizer, the int8 -> bf16
cast, the transposing copy, the autotuned Triton ``tl.dot`` GEMM, the scale and bias kernels.

Stage ``ref`` (a process of its own, only the reference's code on the GPU) writes the full outputs
to a scratch file and times the forward with CUDA events.  Stage ``finish`` (a second process) runs
this repository's layer on the same inputs, compares full outputs, and writes

  * ``ref_w8a16_golden.npz``   the reference's scales (bf16 bits), a SHA-256 of its int8 weights, and
                               the rows ``cases.w8a16_golden_rows`` of every output (bf16 bits);
  * ``ref_w8a16_report.json``  per case: the reference forward's time, and the distance of this
                               repository's CUDA path and of the CPU oracle from the reference's output.

Both files are committed under ``tests/golden/`` and replayed by ``tests/test_golden_w8a16.py`` (CPU:
oracle against the recorded rows) and ``tests/test_gpu_w8a16.py`` (GPU: the kernels against them).

    python tests/golden/make_ref_w8a16_golden.py --out out_dir
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def b16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().copy()


def sha(t):
    return hashlib.sha256(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def tag(outliers):
    return "w8a16_outlier8" if outliers else "w8a16_plain"


def run_ref(work: Path):
    from oracle import build_ref
    from tests.golden import cases

    os.environ.update(build_ref.reference_env())
    sys.path.insert(0, str(build_ref.SITE))
    torch.cuda.init()
    torch.zeros(1, device="cuda")
    t0 = time.time()
    import cublade  # the reference package (import-time warm-up off)
    from cublade.quantization import cuBladeW8A16LinearLayer

    assert Path(cublade.__file__).resolve().is_relative_to(build_ref.SITE.resolve())
    res, timing = {}, {"import_s": round(time.time() - t0, 1)}
    for outliers in (False, True):
        w, cols, bias = cases.w8a16_weight(outliers)
        layer = cuBladeW8A16LinearLayer(cases.W8A16_K, cases.W8A16_N, bias=bias is not None, dtype=torch.bfloat16,
                                        handle_outliers=outliers, outlier_threshold=6.0)
        t0 = time.time()
        layer.quantize(w)
        timing[f"{tag(outliers)}.quantize_s"] = round(time.time() - t0, 2)
        if outliers:
            assert layer.outlier_cols.tolist() == cols, "the weight-side detector picked other columns"
        if bias is not None:
            with torch.no_grad():
                layer.bias.copy_(bias)
        layer = layer.cuda()
        res[f"{tag(outliers)}.int8_weights"] = layer.int8_weights.detach().cpu().numpy().copy()
        res[f"{tag(outliers)}.scales"] = b16(layer.scales)
        for M in cases.W8A16_MS:
            x = cases.w8a16_activations(M, cols).cuda()
            t0 = time.time()
            y = layer(x)
            torch.cuda.synchronize()
            timing[f"{tag(outliers)}.M{M}.first_call_s"] = round(time.time() - t0, 1)
            res[f"{tag(outliers)}.M{M}.y"] = b16(y)
            for _ in range(3):
                layer(x)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(21)]
            ev[0].record()
            for i in range(20):
                layer(x)
                ev[i + 1].record()
            torch.cuda.synchronize()
            ts = sorted(ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(20))
            timing[f"{tag(outliers)}.M{M}.forward_us_median"] = round(ts[10], 1)
            timing[f"{tag(outliers)}.M{M}.forward_us_min"] = round(ts[0], 1)
            print(f"[ref] {tag(outliers)} M={M}: {ts[10]:.1f} us per forward", flush=True)
    np.savez(work / "ref_w8a16_full.npz", **res)
    (work / "ref_w8a16_timing.json").write_text(json.dumps(timing, indent=1))


def finish(work: Path, out: Path):
    import cublade_b200 as cb
    from oracle import oracle as O
    from tests.golden import cases
    from tests.helpers import max_abs_ratio, rel_fro

    full = np.load(work / "ref_w8a16_full.npz")
    timing = json.loads((work / "ref_w8a16_timing.json").read_text())
    gold, report = {}, {"device": torch.cuda.get_device_name(0), "torch": torch.__version__, "timing": timing,
                        "cases": {}}
    try:
        import triton

        report["triton"] = triton.__version__
    except Exception:  # pragma: no cover
        pass
    for outliers in (False, True):
        t = tag(outliers)
        w, cols, bias = cases.w8a16_weight(outliers)
        q_ref = torch.from_numpy(full[f"{t}.int8_weights"])
        s_ref = torch.from_numpy(full[f"{t}.scales"]).view(torch.bfloat16)
        lay = O.w8a16_quantize(w, torch.bfloat16, outlier_cols=cols or None)
        gold[f"{t}.scales"] = full[f"{t}.scales"]
        gold[f"{t}.int8_sha256"] = np.frombuffer(bytes.fromhex(sha(q_ref)), dtype=np.uint8).copy()
        entry = {"int8_weights_ne_oracle": int((q_ref != lay["int8_weights"]).sum()),
                 "scales_ne_oracle": int((s_ref.view(torch.int16) != lay["scales"].view(torch.int16)).sum()),
                 "outlier_cols": cols}
        mine = cb.cuBladeW8A16LinearLayer(cases.W8A16_K, cases.W8A16_N, bias=bias is not None, dtype=torch.bfloat16,
                                          handle_outliers=outliers, outlier_threshold=6.0)
        mine.quantize(w)
        if bias is not None:
            mine.bias = torch.nn.Parameter(bias.clone())
        mine = mine.cuda()
        entry["int8_weights_ne_cuda"] = int((q_ref != mine.int8_weights.cpu()).sum())
        entry["scales_ne_cuda"] = int((s_ref.view(torch.int16) != mine.scales.cpu().view(torch.int16)).sum())
        for M in cases.W8A16_MS:
            x = cases.w8a16_activations(M, cols)
            y_ref = torch.from_numpy(full[f"{t}.M{M}.y"]).view(torch.bfloat16)
            rows = cases.w8a16_golden_rows(M, outliers)
            gold[f"{t}.M{M}.rows"] = np.asarray(rows, dtype=np.int32)
            gold[f"{t}.M{M}.y"] = b16(y_ref[rows])
            gold[f"{t}.M{M}.y_sha256"] = np.frombuffer(bytes.fromhex(sha(y_ref)), dtype=np.uint8).copy()
            y = mine(x.cuda()).cpu()
            y_o = O.w8a16_forward(x[rows], lay, bias)
            entry[f"M{M}"] = {
                "cuda_vs_ref_full": {"rel_fro": rel_fro(y, y_ref), "max_abs_ratio": max_abs_ratio(y, y_ref),
                                     "bf16_bits_ne": int((y.view(torch.int16) != y_ref.view(torch.int16)).sum()),
                                     "n": int(y.numel())},
                "oracle_vs_ref_rows": {"rel_fro": rel_fro(y_o, y_ref[rows]),
                                       "max_abs_ratio": max_abs_ratio(y_o, y_ref[rows]),
                                       "bf16_bits_ne": int((y_o.view(torch.int16) != y_ref[rows].view(torch.int16)).sum()),
                                       "n": int(y_o.numel())},
                "ref_forward_us_median": timing[f"{t}.M{M}.forward_us_median"]}
        report["cases"][t] = entry
    np.savez_compressed(out / "ref_w8a16_golden.npz", **gold)
    (out / "ref_w8a16_report.json").write_text(json.dumps(report, indent=1))
    print(json.dumps(report["cases"], indent=1))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="ref_gpu_out")
    ap.add_argument("--stage", default=None, choices=["ref", "finish"])
    ap.add_argument("--work", default=None)
    a = ap.parse_args()
    out = Path(a.out)
    out.mkdir(exist_ok=True)
    if a.stage == "ref":
        return run_ref(Path(a.work))
    if a.stage == "finish":
        return finish(Path(a.work), out)
    import tempfile

    with tempfile.TemporaryDirectory() as work:
        for st in ("ref", "finish"):
            r = subprocess.run([sys.executable, "-X", "faulthandler", __file__, "--work", work, "--out", str(out),
                                "--stage", st])
            if r.returncode != 0:
                print(f"stage {st} failed with exit code {r.returncode}; stopping")
                sys.exit(1)


if __name__ == "__main__":
    main()
