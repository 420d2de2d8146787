"""Shared helpers for the parity tests."""
from __future__ import annotations

import torch


def bits(t: torch.Tensor) -> torch.Tensor:
    """Raw bit pattern of a tensor as an integer tensor on the CPU (bit-exact comparisons)."""
    t = t.detach().cpu().contiguous()
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8)
    return t


def assert_bits_equal(got: torch.Tensor, want: torch.Tensor, what: str = "") -> None:
    g, w = bits(got), bits(want)
    assert g.shape == w.shape, f"{what}: shape {tuple(g.shape)} != {tuple(w.shape)}"
    if not torch.equal(g, w):
        bad = (g != w).nonzero()
        first = tuple(bad[0].tolist()) if bad.numel() else ()
        raise AssertionError(f"{what}: {bad.shape[0]} of {g.numel()} elements differ, first at {first}: "
                             f"got {g[first].item()} want {w[first].item()}")


def rel_fro(got: torch.Tensor, ref: torch.Tensor) -> float:
    g, r = got.detach().cpu().double(), ref.detach().cpu().double()
    return float((g - r).norm() / r.norm().clamp_min(1e-30))


def max_abs_ratio(got: torch.Tensor, ref: torch.Tensor) -> float:
    g, r = got.detach().cpu().double(), ref.detach().cpu().double()
    return float((g - r).abs().max() / r.abs().max().clamp_min(1e-30))
