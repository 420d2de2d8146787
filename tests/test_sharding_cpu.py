"""World-size-2 ``gloo`` tests (CPU) of the multi-GPU orchestration: shard arithmetic, the single
max-allreduce of per-tensor quantization, and sharded model quantization bookkeeping.  The two
kernels are replaced by the CPU oracle's formulas; what is under test is the host logic."""
import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cublade_b200.sharding import shard_range


def test_shard_range_is_a_balanced_partition():
    for n in (0, 1, 7, 8, 14336, 1 << 20):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_ops():
    from oracle import oracle as O

    def amax_abs(x):
        return x.float().abs().max().reshape(1)

    def cast_per_tensor(x, amax, dtype, eps):
        a = torch.maximum(amax.reshape(()), torch.tensor(eps, dtype=torch.float32))
        if dtype == torch.float8_e4m3fn:
            inv = torch.tensor(448.0) / a
            return (x.float() * inv).to(dtype), torch.tensor(1.0) / inv
        inv = (127.0 / a.double()).float()
        q = torch.round(x.float() * inv).clamp_(-127, 127).to(torch.int8)
        return q, (1.0 / inv.double()).float()

    _ = O
    return SimpleNamespace(amax_abs=amax_abs, cast_per_tensor=cast_per_tensor)


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cublade_b200 import workloads as W
        from cublade_b200.sharding import quantize_tensor_sharded, shard_range
        from oracle import oracle as O

        x = W.fp8_tensor_case(257, 96)  # outliers land on one rank only: the exchange matters
        a, b = shard_range(x.shape[0], rank, world)
        for dtype in (torch.float8_e4m3fn, torch.int8):
            qt = quantize_tensor_sharded(x[a:b].contiguous(), dtype=dtype, ops=_oracle_ops())
            if dtype == torch.float8_e4m3fn:
                q_ref, s_ref = O.fp8_quantize(x)
            else:
                q_ref, s_ref = O.int8_quantize_tensor(x)
            ok_scale = qt.scale.view(torch.int32).item() == s_ref.view(torch.int32).item()
            ok_codes = torch.equal(qt.data.view(torch.uint8), q_ref[a:b].contiguous().view(torch.uint8))
            out.put((rank, str(dtype), ok_scale, ok_codes, qt.mode, qt.original_dtype == x.dtype))
        # column slices of unequal width (7 output features over 2 ranks: 4 + 3) gather back in order
        from cublade_b200.sharding import all_gather_columns

        y = torch.arange(3 * 7, dtype=torch.float32).reshape(3, 7)
        n0, n1 = shard_range(7, rank, world)
        ok_a = torch.equal(all_gather_columns(y[:, n0:n1], out_features=7), y)
        ok_b = torch.equal(all_gather_columns(y[:, n0:n1]), y)  # widths exchanged when out_features is not given
        out.put((rank, "all_gather_columns", ok_a, ok_b, "tensor", True))
    finally:
        dist.destroy_process_group()


def test_sharded_per_tensor_quantization_equals_single_rank_bit_for_bit():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in range(world * 3)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert len(results) == 6
    for rank, dtype, ok_scale, ok_codes, mode, ok_dtype in results:
        assert ok_scale and ok_codes and mode == "tensor" and ok_dtype, (rank, dtype)


class _FakeQuantLayer(torch.nn.Module):
    def __init__(self, in_features, out_features, bias=True, dtype=torch.float32, **kw):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.bias = torch.nn.Parameter(torch.zeros(out_features)) if bias else None
        self.rows = None

    def quantize(self, w):
        self.rows = w.clone()


def test_quantize_model_sharded_gives_each_rank_its_rows(monkeypatch):
    from cublade_b200.quantization import quantizers
    from cublade_b200.sharding import quantize_model_sharded

    quantizers._init_registry()
    monkeypatch.setitem(quantizers.QUANT_LAYER_REGISTRY, "w8a16", _FakeQuantLayer)
    torch.manual_seed(0)
    ref = torch.nn.Sequential(torch.nn.Linear(8, 10), torch.nn.ReLU(), torch.nn.Linear(10, 6, bias=False))
    ref.add_module("lm_head", torch.nn.Linear(6, 4))
    import copy

    world = 4
    shards = [quantize_model_sharded(copy.deepcopy(ref), r, world, exclude_modules=["lm_head"]) for r in range(world)]
    for idx in (0, 2):
        rows = torch.cat([getattr(s, str(idx)).rows for s in shards])
        assert torch.equal(rows, getattr(ref, str(idx)).weight)
        assert sum(getattr(s, str(idx)).out_features for s in shards) == getattr(ref, str(idx)).out_features
    bias = torch.cat([s[0].bias.detach() for s in shards])
    assert torch.equal(bias, ref[0].bias)
    assert all(s[2].bias is None and isinstance(s.lm_head, torch.nn.Linear) for s in shards)
    assert shards[1][0].shard == (1, 4, 3, 6)


def test_an_exchange_object_replaces_the_collective():
    """``quantize_tensor_sharded(..., exchange=ex)`` hands the local amax to ``ex.exchange`` (the peer-memory form on
    GPUs) and does not touch ``torch.distributed``: no process group exists in this test."""
    from cublade_b200.sharding import quantize_tensor_sharded

    seen = []

    class FakeExchange:
        def exchange(self, amax):
            seen.append(float(amax))
            return torch.maximum(amax, torch.tensor([300.0]))  # as if another rank held the maximum

    x = torch.linspace(-2.0, 2.0, 64).to(torch.bfloat16).reshape(8, 8)
    qt = quantize_tensor_sharded(x, dtype=torch.int8, ops=_oracle_ops(), exchange=FakeExchange())
    assert seen == [2.0]
    assert qt.scale.item() == pytest.approx(300.0 / 127.0, rel=1e-6)
    assert int(qt.data.abs().max()) == 1  # 2.0 * 127 / 300 rounds to 1: the foreign maximum set the scale
