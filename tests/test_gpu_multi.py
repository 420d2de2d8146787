"""Multi-GPU parity (needs >= 2 CUDA devices on one node; skipped otherwise).

Ranks are child processes, one per GPU, NCCL backend.  Checked: (1) per-tensor FP8 / INT8
quantization of a row-sharded tensor equals the single-GPU / oracle result bit for bit (one
float32 max-allreduce is the only exchange); (2) a W8A16 layer sharded over its output features
reproduces the unsharded layer's output exactly, slice by slice; (3) the peer-memory form of the exchange
(one small kernel per rank with a bounded wait on its peers' stores) equals the collective.  No rank exits with
work in flight."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cublade_b200 as cb
        from cublade_b200 import workloads as W
        from cublade_b200.sharding import all_gather_columns, quantize_tensor_sharded, shard_range, shard_w8a16_layer
        from oracle import oracle as O

        res = {}
        x = W.fp8_tensor_case(1024, 768)
        a, b = shard_range(x.shape[0], rank, world)
        for dtype, name in ((torch.float8_e4m3fn, "fp8"), (torch.int8, "int8")):
            qt = quantize_tensor_sharded(x[a:b].cuda().contiguous(), dtype=dtype)
            q_ref, s_ref = (O.fp8_quantize(x) if name == "fp8" else O.int8_quantize_tensor(x))
            res[f"{name}_scale"] = qt.scale.cpu().view(torch.int32).item() == s_ref.view(torch.int32).item()
            res[f"{name}_codes"] = torch.equal(qt.data.cpu().view(torch.uint8), q_ref[a:b].contiguous().view(torch.uint8))
            y = cb.dequantize_tensor(qt)
            if name == "fp8":
                want = O.fp8_dequantize(q_ref[a:b], s_ref, x.dtype)
            else:
                want = O.int8_dequantize_rows(q_ref[a:b].reshape(1, -1), s_ref.reshape(1), x.dtype).reshape(b - a, -1)
            res[f"{name}_dequant"] = torch.equal(y.cpu().view(torch.int16), want.view(torch.int16))
        # W8A16 sharded over output features
        w, xa, _ = W.w8a16_case(48, N=1024, K=512)
        full = cb.cuBladeW8A16LinearLayer(512, 1024, bias=True, dtype=torch.bfloat16)
        full.quantize(w)
        full.bias = torch.nn.Parameter(torch.linspace(-1, 1, 1024).to(torch.bfloat16))
        import copy

        mine = shard_w8a16_layer(copy.deepcopy(full), rank, world).cuda()
        y_full = full.cuda()(xa.cuda())
        y_mine = mine(xa.cuda())
        n0, n1 = shard_range(1024, rank, world)
        res["w8a16_slice"] = torch.equal(y_mine, y_full[:, n0:n1])
        res["w8a16_gather"] = torch.equal(all_gather_columns(y_mine), y_full)
        # the same exchange over peer memory (plain peer loads / stores, no multicast): equal to the collective's result
        # on values that differ per rank and per call, and the sharded quantizer built on it gives the same scale
        from cublade_b200 import _native as Nat
        from cublade_b200.sharding import PeerAmaxExchange

        try:
            ex = PeerAmaxExchange()
        except Exception as e:  # symmetric memory is not available on every system: the collective stays the route
            ex, res["peer_exchange_skipped"] = None, True
        if ex is not None:
            g = torch.Generator(device="cuda").manual_seed(17 + rank)
            same = True
            for i in range(25):
                a_loc = (torch.rand(1, generator=g, device="cuda") * 10.0 ** (i % 4)).float()
                want = a_loc.clone()
                dist.all_reduce(want, op=dist.ReduceOp.MAX)
                same = same and torch.equal(ex.exchange(a_loc), want)
            res["peer_exchange_equals_all_reduce"] = same
            qt_peer = quantize_tensor_sharded(x[a:b].cuda().contiguous(), dtype=torch.float8_e4m3fn, exchange=ex)
            q_ref, s_ref = O.fp8_quantize(x)
            res["peer_exchange_fp8_scale"] = qt_peer.scale.cpu().view(torch.int32).item() == s_ref.view(torch.int32).item()
            res["peer_exchange_no_expired_wait"] = Nat.device_error_state() == 0
        torch.cuda.synchronize()
        dist.barrier()
        out.put((rank, res))
    finally:
        dist.destroy_process_group()


def test_sharded_quantization_and_w8a16_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    import torch.multiprocessing as mp

    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, res in results:
        bad = [k for k, v in res.items() if not v]
        assert not bad, f"rank {rank}: {bad}"
