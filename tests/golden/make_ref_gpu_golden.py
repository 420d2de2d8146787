"""Record what the REFERENCE's own CUDA kernels produce on a B200 (run on a GPU box).

Loads the unmodified reference extensions prebuilt in ``oracle/_ref`` (see ``oracle/build_ref.py``),
runs them on the seeded inputs of ``tests/golden/cases.py`` and writes

  * ``ref_gpu_golden.npz``    raw outputs (codes, scale bits, dequantized 16-bit patterns), and
  * ``ref_gpu_report.json``   mismatch counts of those outputs against the CPU oracle on the
                              small cases and on the full-size benchmark configurations,

into the directory given by ``--out``.  The npz is then committed under ``tests/golden/`` and
replayed on the CPU by ``tests/test_golden.py`` -- that is what pins the oracle to the reference.

Each reference extension is exercised in a process of its own (``--stage``), one after the
other: quantizers first, then the dequantizers on the codes the quantizers wrote.

    python tests/golden/make_ref_gpu_golden.py --out out_dir
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

STAGES = ["fp8_quant", "fp8_dequant", "int8_quant", "int8_dequant"]


def u8(t):
    return t.detach().cpu().contiguous().view(torch.uint8).numpy().copy()


def f32bits(t):
    return t.detach().cpu().contiguous().reshape(-1).view(torch.int32).numpy().copy()


def b16(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().copy()


def all_cases():
    from cublade_b200 import workloads as W
    from tests.golden import cases

    fp8 = dict(cases.fp8_cases())
    fp8["big.config1_fp8_4096x4096"] = W.fp8_tensor_case()
    i8t = dict(cases.int8_tensor_cases())
    i8c = dict(cases.int8_channel_cases())
    i8c["big.config2_int8_channel_8192x8192"] = W.int8_channel_case()
    i8g = dict(cases.int8_group_cases())
    i8g["big.config3_int8_group128_4096x8192"] = (W.int8_group_case(rows=4096).view(-1, 128), 128)
    return fp8, i8t, i8c, i8g


def dequantizable(name, i8c):
    """The reference's per-channel dequantizer rejects rows that are not a multiple of 8 long."""
    return name not in i8c or (i8c[name].numel() // i8c[name].shape[0]) % 8 == 0


def run_stage(stage: str, out: Path):
    from oracle.build_ref import load_ref

    fp8, i8t, i8c, i8g = all_cases()
    res = {}
    prev = dict(np.load(out / "ref_stage_quant.npz")) if stage.endswith("dequant") else {}

    def cuda_codes(name, dtype):
        return torch.from_numpy(prev[f"{name}.q"]).view(dtype).cuda()

    def cuda_scale(name, shape):
        return torch.from_numpy(prev[f"{name}.scale"]).view(torch.float32).reshape(shape).cuda()

    if stage == "fp8_quant":
        m = load_ref("cublade_quantize_per_tensor_fp8")
        for name, x in fp8.items():
            q, s = m.quantize_per_tensor_fp8(x.cuda(), 1e-12)
            res[f"{name}.q"], res[f"{name}.scale"] = u8(q), f32bits(s)
    elif stage == "int8_quant":
        m = load_ref("cublade_quantize_int8")
        for name, x in i8t.items():
            q, s = m.quantize_per_tensor_int8(x.cuda(), 1e-12)
            res[f"{name}.q"], res[f"{name}.scale"] = u8(q), f32bits(s)
        for name, x in i8c.items():
            q, s = m.quantize_per_channel_int8(x.cuda(), 1e-12)
            res[f"{name}.q"], res[f"{name}.scale"] = u8(q), f32bits(s)
        for name, (x, G) in i8g.items():
            q, s = m.quantize_per_group_int8(x.cuda(), G, 1e-12)
            res[f"{name}.q"], res[f"{name}.scale"] = u8(q), f32bits(s)
    elif stage == "fp8_dequant":
        m = load_ref("cublade_dequantize_per_tensor_fp8")
        for name in fp8:
            q, s = cuda_codes(name, torch.float8_e4m3fn), cuda_scale(name, ())
            for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
                res[f"{name}.y_{tag}"] = b16(m.dequantize_per_tensor_fp8(q, s, dt))
    elif stage == "int8_dequant":
        m = load_ref("cublade_dequantize_int8")
        for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
            for name in i8t:
                res[f"{name}.y_{tag}"] = b16(m.dequantize_per_tensor_int8(cuda_codes(name, torch.int8),
                                                                          cuda_scale(name, ()), dt))
            for name in i8c:
                if not dequantizable(name, i8c):
                    continue
                res[f"{name}.y_{tag}"] = b16(m.dequantize_per_channel_int8(cuda_codes(name, torch.int8),
                                                                           cuda_scale(name, (-1,)), dt))
            for name, (x, G) in i8g.items():
                res[f"{name}.y_{tag}"] = b16(m.dequantize_per_group_int8(cuda_codes(name, torch.int8),
                                                                         cuda_scale(name, (-1,)), G, dt))
    torch.cuda.synchronize()
    np.savez(out / f"ref_stage_{stage}.npz", **res)
    if stage == "int8_quant":  # both quantizer stages done: merge for the dequantizers
        merged = dict(np.load(out / "ref_stage_fp8_quant.npz"))
        merged.update(res)
        np.savez(out / "ref_stage_quant.npz", **merged)
    print(f"[{stage}] {len(res)} arrays", flush=True)


def finish(work: Path, out: Path):
    """Merge the stages, compare with the CPU oracle, write the golden file and the report."""
    from oracle import oracle as O

    fp8, i8t, i8c, i8g = all_cases()
    got = {}
    for st in STAGES:
        got.update(dict(np.load(work / f"ref_stage_{st}.npz")))

    def ne(a, b):
        return int((np.asarray(a).reshape(-1) != np.asarray(b).reshape(-1)).sum())

    report = {"device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "?", "cases": {}}

    def compare(name, x, q_o, s_o, deq):
        e = {"codes_ne": ne(got[f"{name}.q"], u8(q_o)), "scale_ne": ne(got[f"{name}.scale"], f32bits(s_o)),
             "n": int(x.numel())}
        # dequantized outputs are compared on the REFERENCE's codes and scale
        q_r = torch.from_numpy(got[f"{name}.q"]).view(q_o.dtype).reshape(q_o.shape)
        s_r = torch.from_numpy(got[f"{name}.scale"]).view(torch.float32).reshape(s_o.shape)
        for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
            if f"{name}.y_{tag}" in got:
                e[f"deq_{tag}_ne"] = ne(got[f"{name}.y_{tag}"], b16(deq(q_r, s_r, dt)))
        report["cases"][name] = e

    for name, x in fp8.items():
        q, s = O.fp8_quantize(x)
        compare(name, x, q, s, lambda q, s, dt: O.fp8_dequantize(q, s, dt))
    for name, x in i8t.items():
        q, s = O.int8_quantize_tensor(x)
        compare(name, x, q, s, lambda q, s, dt: O.int8_dequantize_rows(q.reshape(1, -1), s.reshape(1), dt))
    for name, x in i8c.items():
        q, s = O.int8_quantize_channel(x)
        compare(name, x, q, s, lambda q, s, dt: O.int8_dequantize_rows(q.reshape(q.shape[0], -1), s, dt))
    for name, (x, G) in i8g.items():
        q, s = O.int8_quantize_group(x, G)
        compare(name, x, q, s, lambda q, s, dt: O.int8_dequantize_rows(q, s, dt))

    report["total_mismatches"] = sum(v for c in report["cases"].values() for k, v in c.items() if k.endswith("_ne"))
    small = {k: v for k, v in got.items() if not k.startswith("big.")}
    np.savez_compressed(out / "ref_gpu_golden.npz", **small)
    (out / "ref_gpu_report.json").write_text(json.dumps(report, indent=1))
    print(json.dumps({k: v for k, v in report["cases"].items() if k.startswith("big.")}), report["total_mismatches"])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="ref_gpu_out")
    ap.add_argument("--stage", default=None, choices=STAGES)
    ap.add_argument("--work", default=None, help="scratch directory for the per-stage files")
    args = ap.parse_args()
    out = Path(args.out)
    out.mkdir(exist_ok=True)
    if args.stage:
        run_stage(args.stage, Path(args.work))
        return
    import tempfile

    with tempfile.TemporaryDirectory() as work:
        for st in ["fp8_quant", "int8_quant", "fp8_dequant", "int8_dequant"]:
            r = subprocess.run([sys.executable, "-X", "faulthandler", __file__, "--work", work, "--stage", st])
            if r.returncode != 0:
                print(f"stage {st} failed with exit code {r.returncode}; stopping")
                sys.exit(1)
        finish(Path(work), out)


if __name__ == "__main__":
    main()
