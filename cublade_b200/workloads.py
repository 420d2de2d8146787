"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

All tensors are generated on the CPU with an explicit ``torch.Generator`` in float32 and then cast,
so a checker on the host and the kernels on the device see identical bits.  ``rows`` / ``cols``
arguments shrink a configuration for tests; the defaults are the full sizes.
"""
from __future__ import annotations

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def fp8_tensor_case(rows: int = 4096, cols: int = 4096, dtype=torch.bfloat16, n_outliers: int = 16, seed: int = 0):
    """Per-tensor FP8 case: N(0,1)*2 with ``n_outliers`` entries set to +-300 (alternating sign)."""
    g = _gen(seed)
    x = torch.randn(rows, cols, generator=g, dtype=torch.float32) * 2.0
    n = rows * cols
    pos = torch.randperm(n, generator=g)[: min(n_outliers, n)]
    flat = x.view(-1)
    signs = torch.where(torch.arange(pos.numel()) % 2 == 0, 1.0, -1.0)
    flat[pos] = 300.0 * signs
    return x.to(dtype)


def int8_channel_case(rows: int = 8192, cols: int = 8192, dtype=torch.bfloat16, seed: int = 1):
    """Per-channel INT8 case: a weight-like matrix N(0, 0.02)."""
    return (torch.randn(rows, cols, generator=_gen(seed), dtype=torch.float32) * 0.02).to(dtype)


def int8_group_case(rows: int = 16384, cols: int = 8192, dtype=torch.bfloat16, seed: int = 2):
    """Per-group INT8 case: heavy-tailed activations, Student-t with 3 degrees of freedom, times 0.5."""
    g = _gen(seed)
    z = torch.randn(rows, cols, generator=g, dtype=torch.float32)
    chi = torch.zeros(rows, cols, dtype=torch.float32)
    for _ in range(3):
        chi += torch.randn(rows, cols, generator=g, dtype=torch.float32) ** 2
    return (z / torch.sqrt(chi / 3.0) * 0.5).to(dtype)


def w8a16_case(M: int, N: int = 14336, K: int = 4096, dtype=torch.bfloat16, seed: int = 3, n_outlier_cols: int = 0):
    """W8A16 case: weight [N, K] ~ N(0, 0.02) and activations [M, K] ~ N(0, 1).

    With ``n_outlier_cols`` > 0 that many input-feature columns (chosen by the seed) have their
    activations scaled by 20 -- the LLM.int8 scenario; the sorted column list is returned too.
    """
    g = _gen(seed)
    w = (torch.randn(N, K, generator=g, dtype=torch.float32) * 0.02).to(dtype)
    x = torch.randn(M, K, generator=g, dtype=torch.float32)
    cols = []
    if n_outlier_cols:
        cols = sorted(torch.randperm(K, generator=g)[:n_outlier_cols].tolist())
        x[:, cols] *= 20.0
    return w, x.to(dtype), cols


def sharded_fp8_chunk(chunk: int, chunk_elems: int = 1 << 27, dtype=torch.bfloat16, device="cuda", seed: int = 4):
    """Chunk ``chunk`` of the 2^33-element sharded FP8 tensor: N(0,1), generated on ``device`` from a
    seed that depends only on (seed, chunk), so the tensor's content does not depend on how many
    GPUs share it."""
    g = torch.Generator(device=device)
    g.manual_seed(seed * 1_000_003 + chunk)
    return torch.randn(chunk_elems, generator=g, dtype=torch.float32, device=device).to(dtype)
