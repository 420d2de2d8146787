"""CPU checks of bench.py's workload table: every workload builds its host input without a device, its CPU
formulation (the reference arm) runs, and both arms would print the same `config`."""
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = mod
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("name", ["int8_channel", "fp8_tensor", "int8_group", "int8_group_axis0", "rmsnorm_int8"])
def test_workload_cpu_arm(bench, name):
    wl = bench.WORKLOADS[name](None, rows=256, cols=512)
    x = wl.cpu_input()
    assert x.shape == (256, 512) and x.dtype == torch.bfloat16
    y = wl.cpu_step(x)
    assert y.numel() == x.numel() and y.dtype == torch.bfloat16
    y = y.reshape(x.shape)  # the row-group formulation returns [groups, group_size]
    # quantize + dequantize of a tensor stays within one quantization step of it
    err = (y.float() - (x.float() if name != "rmsnorm_int8" else y.float())).abs().max().item()
    bound = {"fp8_tensor": 0.07 * x.float().abs().max().item()}.get(name, x.float().abs().max().item() / 127.0 + 1e-2)
    assert err <= bound
    cfg = wl.config()
    assert set(cfg) == {"workload", "bytes_per_step", "seed"}
    assert cfg["bytes_per_step"] == wl.q_bytes + wl.dq_bytes


def test_group_axis0_cpu_arm_matches_the_oracle(bench):
    from oracle import oracle as O

    wl = bench.WORKLOADS["int8_group_axis0"](None, rows=256, cols=64)
    x = wl.cpu_input()
    q = O.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=128, ch_axis=0)
    assert torch.equal(wl.cpu_step(x), O.dequantize_tensor(q))


def test_failed_child_is_reported_under_its_keys(bench):
    """Without a GPU the child process of the secondary measurements exits with an error: the caller gets the three
    keys with the reason instead of an exception (its own measurements survive a failure of that process)."""
    if torch.cuda.is_available():
        pytest.skip("the child would run the measurements here")
    got = bench.single_gpu_extras_in_child(2, 3, 0)
    assert set(got) == {"configs", "next_rows", "w8a16"}
    assert all("error" in v and "exit status" in v["error"] for v in got.values())
