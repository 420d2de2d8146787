"""Checkpoint round trip of quantized models on the CPU (no kernel runs: the buffers are filled from the CPU
formulation).  The on-disk state is the layers' registered buffers under the reference's names
(cublade/quantization/linear.py:25-33); the quirks covered are the ones that make a plain ``load_state_dict`` fail:
``None`` buffers missing from ``state_dict`` and the narrower ``int8_weights`` of outlier mode (linear.py:66)."""
import pytest
import torch
import torch.nn as nn

from oracle import oracle as O


class Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.embed = nn.Embedding(50, 64)
        self.fc1 = nn.Linear(64, 96)
        self.block = nn.Sequential(nn.Linear(96, 96, bias=False), nn.ReLU())
        self.head = nn.Linear(96, 10)


def _quantized_toy(outliers: bool):
    """A Toy whose fc1 / block.0 are quantized layers with buffers filled from the oracle (CPU only)."""
    import cublade_b200.quantization as Q

    torch.manual_seed(1)
    model = Toy().to(torch.bfloat16)
    with torch.no_grad():
        model.fc1.weight[:, [5, 40]] *= 60.0  # two outlier input features
        model.block[0].weight[:, [7]] *= 60.0
    for parent, leaf in ((model, "fc1"), (model.block, "0")):
        lin = getattr(parent, leaf)
        cols = O.detect_outlier_columns(lin.weight.detach(), 6.0) if outliers else []
        ref = O.w8a16_quantize(lin.weight.detach(), torch.bfloat16, cols if outliers else None)
        layer = Q.cuBladeW8A16LinearLayer(lin.in_features, lin.out_features, bias=lin.bias is not None,
                                          dtype=torch.bfloat16, handle_outliers=outliers)
        layer.int8_weights = ref["int8_weights"]
        layer.scales.copy_(ref["scales"])
        if outliers:
            layer.outlier_weights = ref["outlier_weights"]
            layer.normal_cols = torch.tensor(ref["normal_cols"], dtype=torch.long)
            layer.outlier_cols = torch.tensor(ref["outlier_cols"], dtype=torch.long)
        if lin.bias is not None:
            layer.bias = lin.bias
        setattr(parent, leaf, layer)
    return model


@pytest.mark.parametrize("outliers", [False, True])
def test_round_trip_is_bitwise_and_keys_are_the_references(tmp_path, outliers):
    import cublade_b200.quantization as Q

    model = _quantized_toy(outliers)
    sd = model.state_dict()
    expect = {"fc1.int8_weights", "fc1.scales", "fc1.bias", "block.0.int8_weights", "block.0.scales"}
    if outliers:
        expect |= {f"{p}.{k}" for p in ("fc1", "block.0") for k in ("outlier_weights", "normal_cols", "outlier_cols")}
        assert sd["fc1.int8_weights"].shape == (96, 62)  # narrower: the two outlier columns are kept in 16-bit
    assert {k for k in sd if k.startswith(("fc1", "block"))} == expect

    path = tmp_path / "q.pt"
    Q.save_quantized_model(model, path)
    fresh = Q.load_quantized_model(Toy().to(torch.bfloat16), path)
    assert isinstance(fresh.fc1, Q.cuBladeW8A16LinearLayer) and isinstance(fresh.head, nn.Linear)
    assert fresh.fc1.handle_outliers == outliers
    sd2 = fresh.state_dict()
    assert sd2.keys() == sd.keys()
    for k in sd:
        assert sd2[k].dtype == sd[k].dtype and torch.equal(sd2[k], sd[k]), k
    if not outliers:
        assert fresh.fc1.outlier_weights is None and "fc1.outlier_cols" not in sd2

    # a plain load_state_dict into a freshly built outlier layer is what fails without the helper
    if outliers:
        skeleton = Q.cuBladeW8A16LinearLayer(64, 96, bias=True, dtype=torch.bfloat16, handle_outliers=True)
        with pytest.raises(RuntimeError):
            skeleton.load_state_dict({k[4:]: v for k, v in sd.items() if k.startswith("fc1.")})


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_load_slices_output_features(tmp_path, world):
    import cublade_b200.quantization as Q
    from cublade_b200.sharding import shard_range

    model = _quantized_toy(True)
    path = tmp_path / "q.pt"
    Q.save_quantized_model(model, path)
    full = model.state_dict()
    parts = [Q.load_quantized_model(Toy().to(torch.bfloat16), path, rank=r, world_size=world) for r in range(world)]
    for key in ("int8_weights", "scales", "outlier_weights", "bias"):
        got = torch.cat([p.state_dict()[f"fc1.{key}"] for p in parts], dim=0)
        assert torch.equal(got, full[f"fc1.{key}"]), key
    for r, p in enumerate(parts):
        lo, hi = shard_range(96, r, world)
        assert p.fc1.out_features == hi - lo and p.fc1.shard == (r, world, lo, hi)
        assert torch.equal(p.state_dict()["fc1.outlier_cols"], full["fc1.outlier_cols"])  # replicated
        assert torch.equal(p.state_dict()["head.weight"], full["head.weight"])  # other modules unsharded
    with pytest.raises(ValueError):
        Q.load_quantized_state_dict(model, full, rank=2, world_size=2)


def test_w8a8_layers_and_version_check(tmp_path):
    import cublade_b200.quantization as Q

    model = nn.Sequential(nn.Linear(32, 48), nn.ReLU(), nn.Linear(48, 8)).to(torch.bfloat16)
    ref = O.w8a16_quantize(model[0].weight.detach(), torch.bfloat16)
    layer = Q.cuBladeW8A8LinearLayer(32, 48, bias=True, dtype=torch.bfloat16)
    layer.int8_weights.copy_(ref["int8_weights"])
    layer.scales.copy_(ref["scales"])
    layer.bias = model[0].bias
    model[0] = layer
    path = tmp_path / "q8.pt"
    Q.save_quantized_model(model, path)
    fresh = Q.load_quantized_model(nn.Sequential(nn.Linear(32, 48), nn.ReLU(), nn.Linear(48, 8)).to(torch.bfloat16), path)
    assert isinstance(fresh[0], Q.cuBladeW8A8LinearLayer)
    assert all(torch.equal(a, b) for a, b in zip(fresh.state_dict().values(), model.state_dict().values()))
    blob = torch.load(path, weights_only=True)
    blob["format_version"] = 99
    torch.save(blob, path)
    with pytest.raises(ValueError, match="format_version"):
        Q.load_quantized_model(nn.Sequential(nn.Linear(32, 48), nn.ReLU(), nn.Linear(48, 8)), path)
