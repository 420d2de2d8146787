"""Single-node multi-GPU use of the quantization path: one process per GPU, ``torch.distributed``.

The reference has no multi-GPU code; this module adds only what the path needs.

* Per-channel / per-group quantization and every dequantization shard by rows with NO
  communication: each rank calls the ordinary single-GPU functions on its rows.
* Per-tensor quantization (FP8 or INT8) needs the global amax: each rank reduces its shard
  (``amax_abs``), the ranks max-allreduce ONE float32 (exact and order independent, so the sharded
  result is bit-identical to the single-GPU result), then each rank casts its shard.
* The W8A16 linear shards its output features: per-output-channel scales make the row blocks of
  ``int8_weights`` independent; activations are replicated.
"""
from __future__ import annotations

from types import SimpleNamespace
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .quantization.tensor import QuantizedTensor


def shard_range(n: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous, balanced split of ``n`` rows: the first ``n % world_size`` ranks get one extra row."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(n, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def _native_ops():
    from .bindings.cuda.split_phase import amax_abs, cast_per_tensor

    return SimpleNamespace(amax_abs=amax_abs, cast_per_tensor=cast_per_tensor)


class PeerAmaxExchange:
    """The max-exchange of ``quantize_tensor_sharded`` over NVLink peer memory instead of an NCCL call.

    Built once per process group (all ranks on one node, one GPU each): a 264-byte state array per rank in torch's
    symmetric memory, which maps every rank's array into every process.  ``exchange(local_amax)`` is then one small
    kernel per rank -- a 64-bit store into each peer's array, a bounded wait on the rank's own -- against tens of
    microseconds for a 4-byte all-reduce.  Construction is collective (rendezvous + barrier) and raises where
    symmetric memory is not available; callers fall back to the collective then.
    """

    def __init__(self, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        from .bindings.cuda.split_phase import peer_exchange_state_bytes

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        words = (peer_exchange_state_bytes() + 7) // 8
        self.state = symm_mem.empty(words, dtype=torch.int64, device=device)
        self.state.zero_()
        self.handle = symm_mem.rendezvous(self.state, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world:
            raise RuntimeError("symmetric memory returned a pointer list of another size than the group")
        torch.cuda.synchronize(device)
        dist.barrier(group)  # every rank's array is zero before anybody stores into it

    def exchange(self, local_amax: torch.Tensor) -> torch.Tensor:
        from .bindings.cuda.split_phase import amax_peer_exchange

        return amax_peer_exchange(local_amax, self.ptrs, self.rank)


def quantize_tensor_sharded(x_local: torch.Tensor, dtype: torch.dtype = torch.float8_e4m3fn, eps: float = 1e-12,
                            group=None, ops=None, exchange: Optional["PeerAmaxExchange"] = None) -> QuantizedTensor:
    """Per-tensor quantization of a tensor whose rows are spread over the ranks of ``group``.

    Every rank passes its own contiguous shard and receives the codes of that shard plus the
    (identical on all ranks) global scale.  One exchange: the maximum of a float32 scalar, by ``all_reduce(MAX)`` or,
    with ``exchange`` (a ``PeerAmaxExchange`` built for the same group), by peer-memory stores.
    ``ops`` replaces the two kernels (used by CPU tests of the orchestration).
    """
    import torch.distributed as dist

    ops = ops or _native_ops()
    amax = ops.amax_abs(x_local)
    if exchange is not None:
        amax = exchange.exchange(amax)
    elif dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    q, scale = ops.cast_per_tensor(x_local, amax, dtype, eps)
    zp = torch.zeros((), dtype=torch.float32, device=x_local.device)
    return QuantizedTensor(q, scale, zp, "tensor", 0, 32, dtype, x_local.dtype)


def shard_w8a16_layer(layer, rank: int, world_size: int):
    """Keep only this rank's block of output features of a quantized ``cuBladeW8A16LinearLayer`` (in place).

    ``int8_weights``, ``scales``, ``bias`` and ``outlier_weights`` are sliced along dim 0; the column
    index buffers are unchanged.  The layer then maps ``[..., in] -> [..., out / world_size]``.
    """
    start, stop = shard_range(layer.out_features, rank, world_size)
    layer.int8_weights = layer.int8_weights[start:stop].contiguous()
    layer.scales = layer.scales[start:stop].contiguous()
    if layer.outlier_weights is not None:
        layer.outlier_weights = layer.outlier_weights[start:stop].contiguous()
    if layer.bias is not None:
        layer.bias = nn.Parameter(layer.bias.detach()[start:stop].contiguous(), requires_grad=layer.bias.requires_grad)
    layer.out_features = stop - start
    layer.shard = (rank, world_size, start, stop)
    layer._dev_cache = {}
    return layer


def quantize_model_sharded(model: nn.Module, rank: int, world_size: int, quant_type: str = "w8a16",
                           target_modules: Optional[List[str]] = None, exclude_modules: Optional[List[str]] = None,
                           **quant_kwargs) -> nn.Module:
    """``quantize_model`` where each rank quantizes and keeps only its ``out_features / world_size`` rows
    of every selected ``nn.Linear`` (no communication: per-channel scales are row-local).

    Selection rules are those of ``quantize_model``.  The resulting layers are column-parallel: their
    outputs are this rank's slice of the full output.
    """
    from .quantization.quantizers import QUANT_LAYER_REGISTRY, _init_registry

    _init_registry()
    if quant_type not in QUANT_LAYER_REGISTRY:
        raise ValueError(f"Unknown quant_type '{quant_type}'. Available: {', '.join(QUANT_LAYER_REGISTRY)}")
    layer_cls = QUANT_LAYER_REGISTRY[quant_type]
    exclude_modules = exclude_modules or []

    def walk(module: nn.Module, prefix: str):
        for name, child in list(module.named_children()):
            path = f"{prefix}.{name}" if prefix else name
            if not isinstance(child, nn.Linear):
                walk(child, path)
                continue
            if any(pat in path for pat in exclude_modules):
                continue
            if target_modules is not None and not any(pat in path for pat in target_modules):
                continue
            start, stop = shard_range(child.out_features, rank, world_size)
            with torch.device(child.weight.device):  # buffers live where the weight does
                new = layer_cls(child.in_features, stop - start, bias=child.bias is not None, dtype=child.weight.dtype,
                                **quant_kwargs)
            setattr(module, name, new)
            new.quantize(child.weight.detach()[start:stop])
            if child.bias is not None:
                new.bias = nn.Parameter(child.bias.detach()[start:stop].clone(), requires_grad=False)
            new.shard = (rank, world_size, start, stop)

    walk(model, "")
    return model


def all_gather_columns(y_local: torch.Tensor, group=None, out_features: Optional[int] = None) -> torch.Tensor:
    """Concatenate the ranks' output-feature slices along the last dim.

    The slices of ``shard_range`` differ by one column when ``out_features`` is not a multiple of the world size;
    pass the unsharded ``out_features`` then (each rank's width follows from it).  Without it every rank must hold
    the same width, which is checked."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    if out_features is None:
        widths = torch.tensor([y_local.shape[-1]], dtype=torch.int64, device=y_local.device)
        all_w = [torch.empty_like(widths) for _ in range(world)]
        dist.all_gather(all_w, widths, group=group)
        widths = [int(w.item()) for w in all_w]
    else:
        widths = [(lambda r: r[1] - r[0])(shard_range(out_features, r, world)) for r in range(world)]
    widest = max(widths)
    mine = y_local.contiguous()
    if mine.shape[-1] != widest:  # pad to the widest slice: all_gather wants equal shapes
        pad = torch.zeros(*mine.shape[:-1], widest - mine.shape[-1], dtype=mine.dtype, device=mine.device)
        mine = torch.cat([mine, pad], dim=-1)
    parts = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(parts, mine, group=group)
    return torch.cat([p[..., :w] for p, w in zip(parts, widths)], dim=-1)
