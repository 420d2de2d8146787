"""Seeded small inputs shared by the golden-vector generators and the tests that replay them.

The shapes are the ones the reference's demo scripts exercise
(examples/quantization/quant_dequant_fp8.py:48-58, quant_dequant_int8.py:51-91) plus ragged
sizes that reach the kernels' tail paths.
"""
from __future__ import annotations

import torch


def _g(seed):
    return torch.Generator().manual_seed(seed)


def fp8_cases():
    bf, hf = torch.bfloat16, torch.float16
    single = torch.full((10_000,), 0.01, dtype=bf)
    single[5000] = 99.5
    return {
        "fp8_toy_1_to_8": torch.arange(1, 9, dtype=bf),
        "fp8_single_outlier": single,
        "fp8_tail_2049": torch.randn(2049, generator=_g(10)).to(bf),
        "fp8_random_bf16": (torch.randn(16384, generator=_g(11)) * 3.0).to(bf),
        "fp8_random_fp16": (torch.randn(16384, generator=_g(12)) * 3.0).to(hf),
        "fp8_all_zero": torch.zeros(512, dtype=bf),
        "fp8_small_magnitudes": (torch.randn(4096, generator=_g(13)) * 1e-3).to(bf),
    }


def int8_tensor_cases():
    return {
        "i8t_linspace": torch.linspace(-1, 1, 256).to(torch.bfloat16),
        "i8t_tail_2049": torch.randn(2049, generator=_g(20)).to(torch.bfloat16),
        "i8t_fp16": (torch.randn(8192, generator=_g(21)) * 3.0).to(torch.float16),
        "i8t_fp32_4099": torch.randn(4099, generator=_g(22)),
    }


def int8_channel_cases():
    return {
        "i8c_8x1024": (torch.randn(8, 1024, generator=_g(30)) * 0.02).to(torch.bfloat16),
        "i8c_64x1000_fp16": (torch.randn(64, 1000, generator=_g(31)) * 0.5).to(torch.float16),
        "i8c_16x260_fp32": torch.randn(16, 260, generator=_g(32)) * 0.02,
        "i8c_4x16384": (torch.randn(4, 16384, generator=_g(33)) * 0.02).to(torch.bfloat16),
    }


def int8_group_cases():
    """name -> (grouped [num_groups, G] tensor, G)"""
    return {
        "i8g_1024_g32": ((torch.randn(32, 32, generator=_g(40)) * 2.0).to(torch.bfloat16), 32),
        "i8g_64x256_g128": ((torch.randn(128, 128, generator=_g(41)) * 2.0).to(torch.bfloat16), 128),
        "i8g_g5_scalar": ((torch.randn(256, 5, generator=_g(42)) * 2.0).to(torch.bfloat16), 5),
        "i8g_g4096": ((torch.randn(3, 4096, generator=_g(43)) * 2.0).to(torch.float16), 4096),
        "i8g_fp32_g16": (torch.randn(64, 16, generator=_g(44)), 16),
    }


# ------------------------------------------------------------------------------------------------
# W8A16 linear layer at the benchmark shape (N = 14336, K = 4096), plain and LLM.int8 variants
# ------------------------------------------------------------------------------------------------
W8A16_N, W8A16_K = 14336, 4096
W8A16_MS = (1, 16, 128, 2048)
W8A16_OUTLIER_COLS = 8


def w8a16_weight(outliers: bool):
    """(weight, outlier columns, bias).  Plain: the bf16 N(0, 0.02) weight of the benchmark, no bias.
    LLM.int8 variant: float32 master weights in which every seventh row of 8 seeded columns is 7.5, so
    that the reference's weight-side detector (cublade/quantization/outlier_utils.py:33-35, threshold
    6.0) selects exactly those columns; K - 8 = 4088 keeps float32 rows 16-byte multiples
    (quantize_int8.cu:496-498).  That variant carries a bias, the plain one does not."""
    from cublade_b200 import workloads as W

    w, _, _ = W.w8a16_case(1, N=W8A16_N, K=W8A16_K)
    if not outliers:
        return w, [], None
    g = _g(33)
    cols = sorted(torch.randperm(W8A16_K, generator=g)[:W8A16_OUTLIER_COLS].tolist())
    w32 = w.float()
    w32[:, cols] = torch.where(torch.arange(W8A16_N)[:, None] % 7 == 0, 7.5, w32[:, cols])
    bias = torch.randn(W8A16_N, generator=g).to(torch.bfloat16)
    return w32, cols, bias


def w8a16_activations(M: int, cols=()):
    """bf16 activations [M, K] of the benchmark (``workloads.w8a16_case(M)``: seeded N(0, 1)); the
    columns ``cols`` are scaled by 20 (exact in bf16 up to the rounding of the product)."""
    from cublade_b200 import workloads as W

    _, x, _ = W.w8a16_case(M, N=W8A16_N, K=W8A16_K)
    if len(cols):
        x = x.float()
        x[:, list(cols)] *= 20.0
        x = x.to(torch.bfloat16)
    return x


def w8a16_golden_rows(M: int, outliers: bool):
    """Rows of the [M, N] output kept in the golden file (all of them for M <= 16)."""
    if M <= 16:
        return list(range(M))
    keep = (8 if outliers else 16) if M <= 128 else (8 if outliers else 32)
    return sorted(torch.randperm(M, generator=_g(400 + M))[:keep].tolist())
