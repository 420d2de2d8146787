"""CPU tests of the host-side layer: the C ABI exports, validation order and exception types of
``quantize_tensor`` / ``dequantize_tensor`` / ``quantize_model`` (no kernel is launched here)."""
import re
from pathlib import Path

import pytest
import torch
import torch.nn as nn

import cublade_b200 as cb
from cublade_b200 import _native as N
from cublade_b200.quantization import (detect_outlier_columns, replace_linear_layers, separate_outliers,
                                       split_weights_by_outliers)

ROOT = Path(__file__).resolve().parents[1]


def test_library_loads_and_exports_every_declared_symbol():
    header = (ROOT / "include" / "cublade_b200.h").read_text()
    declared = set(re.findall(r"\b(cb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    lib = N.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(N.SIGNATURES), "ctypes table and header disagree"
    assert lib.cb_version() >= 100
    assert lib.cb_last_error() is not None
    assert lib.cb_launch_count() == 0  # nothing may have been launched in a CPU-only process


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", tmp_path / "libcublade_b200.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        N.lib()


def test_public_names_match_the_reference_api():
    from cublade_b200 import quantization as Q

    for name in ("quantize_model", "quantize_tensor", "dequantize_tensor", "QuantizedTensor",
                 "cuBladeW8A16LinearLayer", "detect_outlier_columns", "separate_outliers",
                 "split_weights_by_outliers"):
        assert name in Q.__all__ and hasattr(Q, name)
    assert Q.cubladeW8A16LinearLayer is Q.cuBladeW8A16LinearLayer
    import inspect

    sig = inspect.signature(Q.quantize_tensor)
    assert list(sig.parameters) == ["x", "scheme", "dtype", "mode", "group_size", "ch_axis", "eps"]
    assert sig.parameters["group_size"].default == 32 and sig.parameters["eps"].default == 1e-12
    fields = [f for f in Q.QuantizedTensor.__dataclass_fields__]
    assert fields == ["data", "scale", "zero_point", "mode", "axis", "group_size", "dtype", "original_dtype"]


def test_quantize_tensor_validation_order_on_cpu_tensors():
    x = torch.randn(4, 8)
    with pytest.raises(NotImplementedError, match="symmetric"):
        cb.quantize_tensor(x, scheme="affine")
    with pytest.raises(ValueError, match="No quant kernel registered"):
        cb.quantize_tensor(x, dtype=torch.float8_e4m3fn, mode="group")
    with pytest.raises(ValueError, match="No quant kernel registered"):
        cb.quantize_tensor(x, dtype=torch.int8, mode="rowwise")
    with pytest.raises(ValueError, match="must be on CUDA"):
        cb.quantize_tensor(x, dtype=torch.int8, mode="tensor")
    qt = cb.QuantizedTensor(torch.zeros(4, 8, dtype=torch.int8), torch.ones(()), torch.zeros(()), "tensor", 0, 32,
                            torch.int8, torch.bfloat16)
    with pytest.raises(ValueError, match="must be on CUDA"):
        cb.dequantize_tensor(qt)


def test_outlier_utilities():
    w = torch.zeros(6, 10)
    w[2, 3], w[5, 7], w[0, 9] = 6.5, -9.0, 6.0  # 6.0 is not above the threshold
    cols = detect_outlier_columns(w, 6.0)
    assert cols == [3, 7]
    wn, wo, nc, oc = split_weights_by_outliers(w, cols)
    assert nc == [0, 1, 2, 4, 5, 6, 8, 9] and oc == [3, 7]
    assert wn.shape == (6, 8) and wo.shape == (6, 2) and torch.equal(wo, w[:, [3, 7]])
    wn2, wo2, nc2, oc2 = separate_outliers(w, 6.0)
    assert torch.equal(wn, wn2) and oc2 == oc and nc2 == nc
    _, wo3, _, oc3 = split_weights_by_outliers(w, [7, 3])  # explicit list order is kept
    assert oc3 == [7, 3] and torch.equal(wo3, w[:, [7, 3]])
    assert detect_outlier_columns(torch.ones(3, 3)) == []


def test_outlier_utilities_equal_the_reference_module_on_random_weights():
    """The reference's outlier_utils.py is pure torch: loaded by file path from a checkout beside this repository
    (skipped where there is none) and compared call for call on random weights with planted > threshold entries."""
    import importlib.util
    from pathlib import Path

    src = Path(__file__).resolve().parents[2] / "reference" / "cublade" / "quantization" / "outlier_utils.py"
    if not src.exists():
        pytest.skip("no reference checkout beside the repository")
    spec = importlib.util.spec_from_file_location("ref_outlier_utils", src)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    g = torch.Generator().manual_seed(17)
    for shape, thr, planted in (((64, 96), 6.0, 5), ((128, 40), 3.5, 0), ((7, 512), 6.0, 31), ((16, 16), 0.5, 16)):
        w = torch.randn(*shape, generator=g)
        cols = torch.randperm(shape[1], generator=g)[:planted]
        rows = torch.randint(0, shape[0], (planted,), generator=g)
        w[rows, cols] = (thr + 1.0) * torch.where(torch.rand(planted, generator=g) < 0.5, -1.0, 1.0)
        assert detect_outlier_columns(w, thr) == ref.detect_outlier_columns(w, thr)
        mine, theirs = separate_outliers(w, thr), ref.separate_outliers(w, thr)
        assert mine[2] == theirs[2] and mine[3] == theirs[3]
        assert torch.equal(mine[0], theirs[0]) and torch.equal(mine[1], theirs[1])
        explicit = cols.tolist()[::-1]
        a, b = split_weights_by_outliers(w, explicit), ref.split_weights_by_outliers(w, explicit)
        assert a[2] == b[2] and a[3] == b[3] and torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


class _Recorder(nn.Module):
    """Stand-in quantized layer that records how replace_linear_layers drives it."""

    def __init__(self, in_features, out_features, bias=True, dtype=torch.float32, **kw):
        super().__init__()
        self.args = (in_features, out_features, bias, dtype, kw)
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        self.seen = None

    def quantize(self, w):
        self.seen = w


def test_replace_linear_layers_selection_and_bias_handling():
    model = nn.Sequential()
    model.add_module("attn", nn.ModuleDict({"q_proj": nn.Linear(8, 8), "k_proj": nn.Linear(8, 4, bias=False)}))
    model.add_module("mlp", nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 8)))
    model.add_module("lm_head", nn.Linear(8, 32))
    orig_q_bias = model.attn["q_proj"].bias
    orig_q_weight = model.attn["q_proj"].weight
    replace_linear_layers(model, _Recorder, exclude_modules=["lm_head"], quant_kwargs={"handle_outliers": True})
    assert isinstance(model.lm_head, nn.Linear)
    q = model.attn["q_proj"]
    assert isinstance(q, _Recorder) and q.args == (8, 8, True, torch.float32, {"handle_outliers": True})
    assert q.seen is orig_q_weight and q.bias is orig_q_bias  # the original Parameter objects are handed over
    assert model.attn["k_proj"].args[2] is False and model.attn["k_proj"].bias is None
    assert isinstance(model.mlp[0], _Recorder) and isinstance(model.mlp[2], _Recorder)
    m2 = nn.Sequential(nn.Linear(4, 4), nn.Sequential(nn.Linear(4, 4)))
    replace_linear_layers(m2, _Recorder, target_modules=["1.0"])
    assert isinstance(m2[0], nn.Linear) and isinstance(m2[1][0], _Recorder)


def test_quantize_model_registry_errors_and_copy_semantics(monkeypatch):
    from cublade_b200.quantization import quantizers

    with pytest.raises(ValueError, match="Unknown quant_type 'w2a16'. Available: w4a16, w8a16, w8a8"):
        cb.quantize_model(nn.Linear(4, 4), "w2a16")
    monkeypatch.setitem(quantizers.QUANT_LAYER_REGISTRY, "w8a16", _Recorder)
    model = nn.Sequential(nn.Linear(4, 4))
    out = cb.quantize_model(model, "w8a16", inplace=False)
    assert out is not model and isinstance(model[0], nn.Linear) and isinstance(out[0], _Recorder)
    out2 = cb.quantize_model(model, "w8a16")
    assert out2 is model and isinstance(model[0], _Recorder)


def test_w8a16_layer_buffers_and_state_dict_layout():
    layer = cb.cuBladeW8A16LinearLayer(32, 16, bias=True, dtype=torch.bfloat16)
    assert layer.int8_weights.shape == (16, 32) and layer.int8_weights.dtype == torch.int8
    assert layer.scales.shape == (16,) and layer.scales.dtype == torch.bfloat16
    assert layer.outlier_weights is None and layer.normal_cols is None and layer.outlier_cols is None
    assert set(layer.state_dict()) == {"bias", "int8_weights", "scales"}  # None buffers are not serialised
    assert cb.cuBladeW8A16LinearLayer(32, 16, bias=False).bias is None
    with pytest.raises(ValueError, match="CUDA"):
        layer(torch.zeros(2, 32, dtype=torch.bfloat16))


def test_rmsnorm_quantize_oracle_known_answers_and_cpu_rejection():
    """Hand-checked rows for the CPU formulation of the fused RMSNorm -> quantize op, and the wrapper's
    refusal of CPU tensors (there is no CPU path)."""
    import pytest
    import torch

    from oracle import oracle as O
    from cublade_b200.quantization import rmsnorm_quantize_tensor

    x = torch.tensor([[3.0, 4.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0]], dtype=torch.bfloat16)  # mean(x^2) = 25/8
    q, s, y, r = O.rmsnorm_quantize(x, None, rms_eps=0.0)
    assert abs(r.item() - (8.0 / 25.0) ** 0.5) < 1e-7
    assert y.tolist() == [[torch.tensor(3.0 * r.item()).to(torch.bfloat16).item(),
                           torch.tensor(4.0 * r.item()).to(torch.bfloat16).item(), 0, 0, 0, 0, 0, 0]]
    assert q.tolist()[0][:2] == [95, 127] and q.tolist()[0][2:] == [0] * 6  # 3/4 * 127 = 95.25
    gain = torch.tensor([2.0, 0.5, 1, 1, 1, 1, 1, 1], dtype=torch.bfloat16)
    q2, s2, y2, _ = O.rmsnorm_quantize(x, gain, rms_eps=0.0)
    assert y2[0, 0].item() == 2 * y[0, 0].item() and y2[0, 1].item() == 0.5 * y[0, 1].item()
    assert q2.tolist()[0][:2] == [127, 42]  # (4/2) / (3*2) * 127 = 42.33
    qf, sf, _, _ = O.rmsnorm_quantize(x, None, rms_eps=0.0, code=torch.float8_e4m3fn)
    assert qf.float().tolist()[0][:2] == [320.0, 448.0]  # 336 ties to the even neighbour 320
    with pytest.raises(ValueError):
        rmsnorm_quantize_tensor(x)
