"""CPU tests that pin the W8A16 part of the oracle to the reference's own layer.

``tests/golden/ref_w8a16_golden.npz`` holds what the reference's ``cuBladeW8A16LinearLayer``
(``quantize()`` + ``forward()``, unmodified, imported from an install of the reference) produced on
a B200 for the seeded benchmark-shape inputs of ``tests/golden/cases.py``: N = 14336, K = 4096,
M in {1, 16, 128, 2048}, plain and with 8 outlier columns + bias.
``tests/golden/make_ref_w8a16_golden.py`` recorded it; ``ref_w8a16_report.json`` keeps that run's
own comparisons (full outputs) and the reference forward's timings.

Asserted here:
  * the int8 weights (by SHA-256) and the bf16 scales the reference stored equal the oracle's bit for bit;
  * ``oracle.w8a16_forward`` on the recorded rows is inside the stated tolerance (relative Frobenius
    error <= 1e-2, max |err| <= 2e-2 max |ref|) and, beyond that, differs from the reference in fewer
    than 0.2 % of the bf16 values -- what the different order of the fp32 accumulation leaves.
"""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.golden import cases
from tests.helpers import max_abs_ratio, rel_fro

GOLD = Path(__file__).parent / "golden"
REL_FRO_TOL, MAX_ABS_TOL, BITS_NE_FRACTION = 1e-2, 2e-2, 2e-3


@pytest.fixture(scope="module")
def gold():
    return dict(np.load(GOLD / "ref_w8a16_golden.npz"))


@pytest.fixture(scope="module", params=[False, True], ids=["plain", "outlier8"])
def variant(request):
    outliers = request.param
    w, cols, bias = cases.w8a16_weight(outliers)
    return ("w8a16_outlier8" if outliers else "w8a16_plain"), outliers, cols, bias, \
        O.w8a16_quantize(w, torch.bfloat16, outlier_cols=cols or None)


def test_stored_weights_and_scales_equal_the_reference(gold, variant):
    tag, _, _, _, lay = variant
    digest = hashlib.sha256(lay["int8_weights"].contiguous().view(torch.uint8).numpy().tobytes()).digest()
    assert digest == gold[f"{tag}.int8_sha256"].tobytes(), "int8 weights differ from the reference layer's"
    assert np.array_equal(lay["scales"].view(torch.int16).numpy(), gold[f"{tag}.scales"]), "scales differ"


@pytest.mark.parametrize("M", cases.W8A16_MS)
def test_oracle_forward_against_recorded_reference_rows(gold, variant, M):
    tag, outliers, cols, bias, lay = variant
    rows = cases.w8a16_golden_rows(M, outliers)
    assert rows == gold[f"{tag}.M{M}.rows"].tolist()
    y_ref = torch.from_numpy(gold[f"{tag}.M{M}.y"]).view(torch.bfloat16)
    x = cases.w8a16_activations(M, cols)[rows]
    y = O.w8a16_forward(x, lay, bias)
    assert rel_fro(y, y_ref) <= REL_FRO_TOL and max_abs_ratio(y, y_ref) <= MAX_ABS_TOL
    ne = int((y.view(torch.int16) != y_ref.view(torch.int16)).sum())
    assert ne <= BITS_NE_FRACTION * y.numel(), f"{ne} of {y.numel()} bf16 values differ from the reference"


def test_report_of_the_recording_run_is_consistent():
    rep = json.loads((GOLD / "ref_w8a16_report.json").read_text())
    assert rep["device"].startswith("NVIDIA B200")
    for tag in ("w8a16_plain", "w8a16_outlier8"):
        e = rep["cases"][tag]
        assert e["int8_weights_ne_oracle"] == 0 and e["scales_ne_oracle"] == 0
        assert e["int8_weights_ne_cuda"] == 0 and e["scales_ne_cuda"] == 0
        for M in cases.W8A16_MS:
            c = e[f"M{M}"]["cuda_vs_ref_full"]
            assert c["rel_fro"] <= REL_FRO_TOL and c["max_abs_ratio"] <= MAX_ABS_TOL
