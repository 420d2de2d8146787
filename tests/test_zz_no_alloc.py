"""GPU test of ``cb_w8a16_linear_outlier_static``, the LLM.int8 W8A16 entry point for callers that
cannot allocate device memory (its scratch is a fixed array inside the library's device image).

It is called through the raw C ABI and must give exactly what the ordinary route gives
(``cb_gather_columns`` into caller-owned buffers + ``cb_w8a16_linear``), on two calls in a row with
different inputs -- the second call finds the first call's data in the shared scratch.  Requests
larger than the scratch are refused with a clear error and launch nothing.  The file name sorts
last so a run that stops at the first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(M, N, K, KO, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).to(dtype).cuda()
    cols = torch.randperm(K, generator=g)
    outlier = cols[:KO].sort().values.cuda()
    normal = cols[KO:].sort().values.cuda()
    wq = torch.randint(-127, 128, (N, K - KO), generator=g, dtype=torch.int8).cuda()
    scales = (torch.rand(N, generator=g) * 0.01 + 1e-3).to(dtype).cuda()
    bias = torch.randn(N, generator=g).to(dtype).cuda()
    wo = torch.randn(N, max(KO, 1), generator=g).to(dtype).cuda()[:, :KO].contiguous()
    return x, normal, outlier, wq, scales, bias, wo


def _ordinary(x, normal, outlier, wq, scales, bias, wo):
    from cublade_b200.bindings.w8a16 import gather_columns, w8a16_linear

    if outlier.numel() == 0:
        return w8a16_linear(gather_columns(x, normal), wq, scales, bias)
    return w8a16_linear(gather_columns(x, normal), wq, scales, bias, gather_columns(x, outlier), wo)


def _static(x, normal, outlier, wq, scales, bias, wo):
    from cublade_b200 import _native as N

    L = N.lib()
    M, K = x.shape
    y = torch.full((M, wq.shape[0]), float("nan"), dtype=x.dtype, device=x.device)
    st = L.cb_w8a16_linear_outlier_static(
        x.data_ptr(), M, K, x.stride(0), normal.data_ptr(), outlier.data_ptr(), outlier.numel(), wq.data_ptr(),
        wq.shape[0], scales.data_ptr(), N.dtype_code(scales.dtype), bias.data_ptr(), N.dtype_code(bias.dtype),
        wo.data_ptr(), y.data_ptr(), y.stride(0), N.dtype_code(x.dtype), torch.cuda.current_stream().cuda_stream)
    return st, y


def test_static_scratch_entry_point_matches_ordinary_route_twice_and_rejects_oversize():
    from cublade_b200 import _native as N

    L = N.lib()
    assert L.cb_static_scratch_bytes() == 16 << 20
    # two calls in a row, different shapes and data; the second one is larger than the first
    for M, Nout, K, KO, seed in ((7, 96, 520, 8, 1), (150, 384, 1032, 8, 2)):
        prob = _problem(M, Nout, K, KO, seed)
        want = _ordinary(*prob)
        status, got = _static(*prob)
        torch.cuda.synchronize()
        assert status == 0, L.cb_static_last_error()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"M={M}: outputs differ"
    assert N.device_error_state() == 0
    # the other routes behind the entry point: float16; K - KO not a multiple of 8 (padded row stride of the
    # re-packed activations, generic streaming kernel); no outlier columns at all; and a shape whose
    # tensor-core schedule splits K and takes its workspace from the tail of the built-in array
    for M, Nout, K, KO, seed, dtype in ((5, 64, 523, 3, 4, torch.float16), (40, 128, 1029, 5, 5, torch.bfloat16),
                                        (9, 48, 256, 0, 6, torch.bfloat16), (64, 2048, 8200, 8, 7, torch.bfloat16)):
        prob = _problem(M, Nout, K, KO, seed, dtype)
        want = _ordinary(*prob)
        before = N.launch_count()
        status, got = _static(*prob)
        torch.cuda.synchronize()
        assert status == 0, L.cb_static_last_error()
        assert N.launch_count() - before >= (3 if KO else 2), "the entry point accounts for its launches"
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"M={M} K={K} KO={KO} {dtype}: outputs differ"
    assert L.cb_w8a16_workspace_bytes(64, 2048, 8192) > 0, "shape chosen so that the split round is planned"
    assert N.device_error_state() == 0
    # argument checks the ordinary entry point makes too: dtype codes and row strides
    prob = _problem(4, 16, 64, 8, 8)
    x, normal, outlier, wq, scales, bias, wo = prob
    y = torch.full((4, 16), 3.0, dtype=torch.bfloat16, device="cuda")
    args = lambda sdt, ldx, ldy: (x.data_ptr(), 4, 64, ldx, normal.data_ptr(), outlier.data_ptr(), 8, wq.data_ptr(), 16,  # noqa: E731
                                  scales.data_ptr(), sdt, bias.data_ptr(), N.CB_BF16, wo.data_ptr(), y.data_ptr(), ldy,
                                  N.CB_BF16, torch.cuda.current_stream().cuda_stream)
    assert L.cb_w8a16_linear_outlier_static(*args(9, 64, 16)) == 2   # CB_ERR_DTYPE
    assert L.cb_w8a16_linear_outlier_static(*args(N.CB_BF16, 63, 16)) == 1  # CB_ERR_ARGUMENT: ldx < K
    assert L.cb_w8a16_linear_outlier_static(*args(N.CB_BF16, 64, 15)) == 1  # CB_ERR_ARGUMENT: ldy < N
    torch.cuda.synchronize()
    assert bool((y == 3.0).all())
    # beyond the built-in scratch: refused before anything is launched, output untouched
    M, K = 4096, 4096  # 4096 * 4096 * 2 B = 32 MiB > 16 MiB
    x = torch.zeros(M, K, dtype=torch.bfloat16, device="cuda")
    small = _problem(4, 16, 64, 8, 3)
    launches = N.launch_count()
    y = torch.full((M, 16), 3.0, dtype=torch.bfloat16, device="cuda")
    st = L.cb_w8a16_linear_outlier_static(
        x.data_ptr(), M, K, K, small[1].data_ptr(), small[2].data_ptr(), 8, small[3].data_ptr(), 16,
        small[4].data_ptr(), N.CB_BF16, None, 0, small[6].data_ptr(), y.data_ptr(), 16, N.CB_BF16,
        torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == 4  # CB_ERR_RANGE
    assert b"scratch" in L.cb_static_last_error()
    assert N.launch_count() == launches and bool((y == 3.0).all())
