"""GPU parity: the sm_100a kernels (called through the C ABI via the binding layer) against the
CPU oracle, bit for bit.  Shapes follow the reference's demo scripts
(examples/quantization/quant_dequant_fp8.py:48-58, quant_dequant_int8.py:51-91) plus the
benchmark configurations at full size."""
import ctypes

import pytest
import torch

from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _cuda(t):
    return t.to("cuda").contiguous()


def _fp8_cases():
    g = torch.Generator().manual_seed(0)
    bf = torch.bfloat16
    single = torch.full((10_000,), 0.01, dtype=bf)
    single[5000] = 99.5
    return [
        ("toy_1_to_8", torch.arange(1, 9, dtype=bf)),
        ("1M_random", (torch.randn(1_000_000, generator=g) * 3.0).to(bf)),
        ("single_outlier", single),
        ("tail_2049", torch.randn(2049, generator=g).to(bf)),
        ("fp16_parity", (torch.randn(1_000_000, generator=g) * 3.0).to(torch.float16)),
        ("all_zero", torch.zeros(4096, dtype=bf)),
        ("one_element", torch.tensor([-3.5], dtype=bf)),
        ("tiny_values", (torch.randn(5000, generator=g) * 1e-20).to(bf)),
        ("3d_shape", torch.randn(3, 17, 33, generator=g).to(bf)),
    ]


@pytest.mark.parametrize("name,x", _fp8_cases(), ids=[c[0] for c in _fp8_cases()])
def test_fp8_roundtrip_demo_shapes(name, x):
    import cublade_b200 as cb

    qt = cb.quantize_tensor(_cuda(x), dtype=torch.float8_e4m3fn, mode="tensor")
    q_ref, s_ref = O.fp8_quantize(x)
    assert qt.data.dtype == torch.float8_e4m3fn and qt.data.shape == x.shape
    assert qt.scale.shape == () and qt.scale.dtype == torch.float32
    assert_bits_equal(qt.scale, s_ref, f"{name} scale")
    assert_bits_equal(qt.data, q_ref, f"{name} codes")
    y = cb.dequantize_tensor(qt)
    assert y.dtype == x.dtype
    assert_bits_equal(y, O.fp8_dequantize(q_ref, s_ref, x.dtype), f"{name} dequant")


def test_fp8_config1_full_size_and_both_output_types():
    from cublade_b200 import workloads as W
    from cublade_b200.bindings.cuda import dequantize_per_tensor_fp8, quantize_per_tensor_fp8

    x = W.fp8_tensor_case()  # 4096 x 4096, 16 outliers of magnitude 300
    q, s = quantize_per_tensor_fp8(_cuda(x))
    q_ref, s_ref = O.fp8_quantize(x)
    assert s_ref.item() == pytest.approx(0.66964287, rel=1e-7)
    assert_bits_equal(s, s_ref, "scale")
    assert_bits_equal(q, q_ref, "codes")
    for dt in (torch.bfloat16, torch.float16):
        assert_bits_equal(dequantize_per_tensor_fp8(q, s, dt), O.fp8_dequantize(q_ref, s_ref, dt), f"dequant {dt}")


@pytest.mark.parametrize("n", [1, 7, 8, 9, 2047, 2048, 2049, 262_144 + 3])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_int8_per_tensor_sizes(n, dtype):
    from cublade_b200.bindings.cuda import dequantize_per_tensor_int8, quantize_per_tensor_int8

    x = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 1.7).to(dtype)
    q, s = quantize_per_tensor_int8(_cuda(x))
    q_ref, s_ref = O.int8_quantize_tensor(x)
    assert_bits_equal(s, s_ref, "scale")
    assert_bits_equal(q, q_ref, "codes")
    for dt in (torch.bfloat16, torch.float16):
        want = O.int8_dequantize_rows(q_ref.reshape(1, -1), s_ref.reshape(1), dt).reshape(x.shape)
        assert_bits_equal(dequantize_per_tensor_int8(q, s, dt), want, f"dequant {dt}")


def test_int8_per_tensor_linspace_toy():
    import cublade_b200 as cb

    x = torch.linspace(-1, 1, 256).to(torch.bfloat16)
    qt = cb.quantize_tensor(_cuda(x), dtype=torch.int8, mode="tensor")
    assert qt.scale.item() == pytest.approx(0.0078740157, rel=1e-7)
    assert qt.data[:10].tolist() == list(range(-127, -117))
    assert_bits_equal(qt.data, O.int8_quantize_tensor(x)[0], "codes")


@pytest.mark.parametrize("shape", [(8, 1024), (1024, 1024), (4096, 4096), (3, 8), (5, 24), (7, 1000), (33, 2056),
                                   (2, 4, 16), (6, 16384), (4, 16392), (3, 40000)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_int8_per_channel(shape, dtype):
    import cublade_b200 as cb

    if dtype == torch.float32 and shape == (4096, 4096):
        pytest.skip("covered by the 16-bit variants")
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.randn(*shape, generator=g) * 0.02).to(dtype)
    x[0].zero_()  # an all-zero channel exercises the eps floor
    qt = cb.quantize_tensor(_cuda(x), dtype=torch.int8, mode="channel", ch_axis=0)
    ref = O.quantize_tensor(x, torch.int8, "channel")
    assert qt.scale.shape == (shape[0],)
    assert_bits_equal(qt.scale, ref["scale"], "scales")
    assert_bits_equal(qt.data, ref["data"], "codes")
    if dtype != torch.float32:
        assert_bits_equal(cb.dequantize_tensor(qt), O.dequantize_tensor(ref), "dequant")


def test_int8_per_channel_config2_full_size():
    from cublade_b200 import workloads as W
    from cublade_b200.bindings.cuda import dequantize_per_channel_int8, quantize_per_channel_int8

    x = W.int8_channel_case()  # 8192 x 8192
    q, s = quantize_per_channel_int8(_cuda(x))
    q_ref, s_ref = O.int8_quantize_channel(x)
    assert_bits_equal(s, s_ref, "scales")
    assert_bits_equal(q, q_ref, "codes")
    amax = x.float().abs().amax(dim=1)
    assert int((s_ref != amax / 127.0).sum()) > 1000  # the kernel formula, not amax/127
    y = dequantize_per_channel_int8(q, s, torch.bfloat16)
    assert_bits_equal(y, O.int8_dequantize_rows(q_ref, s_ref, torch.bfloat16), "dequant")


@pytest.mark.parametrize("shape,G,axis", [((1024,), 32, 0), ((1024, 1024), 128, -1), ((512, 4096), 32, -1),
                                          ((64, 96), 8, -1), ((64, 96), 16, 1), ((96, 64), 32, 0), ((4, 8192), 4096, -1),
                                          ((40, 35), 5, -1), ((16, 300), 100, -1), ((8, 6, 64), 64, 2),
                                          ((8, 64, 6), 16, 1), ((3, 2000), 1000, -1)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_int8_per_group(shape, G, axis, dtype):
    import cublade_b200 as cb

    g = torch.Generator().manual_seed(G + len(shape))
    x = (torch.randn(*shape, generator=g) * 2.0).to(dtype)
    qt = cb.quantize_tensor(_cuda(x), dtype=torch.int8, mode="group", group_size=G, ch_axis=axis)
    ref = O.quantize_tensor(x, torch.int8, "group", group_size=G, ch_axis=axis)
    assert qt.scale.shape == ref["scale"].shape and qt.data.shape == x.shape
    assert_bits_equal(qt.scale, ref["scale"], "scales")
    assert_bits_equal(qt.data, ref["data"], "codes")
    if dtype != torch.float32:
        assert_bits_equal(cb.dequantize_tensor(qt), O.dequantize_tensor(ref), "dequant")


def test_int8_per_group_config3_scaled_and_fp16_legacy_dequant():
    from cublade_b200 import workloads as W
    from cublade_b200.bindings.cuda import dequantize_per_group_int8, quantize_per_group_int8

    x = W.int8_group_case(rows=2048)  # 2048 x 8192 heavy-tailed, same distribution as the full case
    xg = x.view(-1, 128)
    q, s = quantize_per_group_int8(_cuda(xg), 128)
    q_ref, s_ref = O.int8_quantize_group(xg, 128)
    assert_bits_equal(s, s_ref, "scales")
    assert_bits_equal(q, q_ref, "codes")
    for dt in (torch.bfloat16, torch.float16):
        assert_bits_equal(dequantize_per_group_int8(q, s, 128, dt), O.int8_dequantize_rows(q_ref, s_ref, dt),
                          f"dequant {dt}")


def test_outputs_stay_inside_their_buffers():
    """Canary bands around every output written through the raw C ABI, odd sizes included."""
    from cublade_b200 import _native as N

    L = N.lib()
    pad = 256
    stream = torch.cuda.current_stream().cuda_stream
    for n in (1, 9, 2049, 70_001):
        x = (torch.randn(n, generator=torch.Generator().manual_seed(n)) * 3).to(torch.bfloat16).cuda()
        qbuf = torch.full((n + 2 * pad,), 0x5A, dtype=torch.uint8, device="cuda")
        sbuf = torch.full((3,), 7.25, dtype=torch.float32, device="cuda")
        amax = torch.empty(N.per_tensor_scratch_floats(), dtype=torch.float32, device="cuda")
        N.check(L.cb_quantize_per_tensor_fp8(x.data_ptr(), N.CB_BF16, n, 1e-12, qbuf.data_ptr() + pad,
                                             sbuf.data_ptr() + 4, amax.data_ptr(), stream))
        torch.cuda.synchronize()
        assert (qbuf[:pad] == 0x5A).all() and (qbuf[pad + n:] == 0x5A).all()
        assert sbuf[0].item() == 7.25 and sbuf[2].item() == 7.25
        q_ref, s_ref = O.fp8_quantize(x.cpu())
        assert_bits_equal(qbuf[pad:pad + n].cpu(), q_ref.view(torch.uint8), "codes")
        ybuf = torch.full((n + 2 * pad,), -1.0, dtype=torch.bfloat16, device="cuda")
        N.check(L.cb_dequantize_per_tensor_fp8(qbuf.data_ptr() + pad, sbuf.data_ptr() + 4, n, N.CB_BF16,
                                               ybuf.data_ptr() + 2 * pad, stream))
        torch.cuda.synchronize()
        assert (ybuf[:pad] == -1).all() and (ybuf[pad + n:] == -1).all()
        assert_bits_equal(ybuf[pad:pad + n], O.fp8_dequantize(q_ref, s_ref, torch.bfloat16), "dequant")
    # per-group with a misaligned base pointer takes the scalar kernels
    G, rows = 24, 37
    x = torch.randn(rows * G + 1, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
    qbuf = torch.full((rows * G + 2 * pad,), 0x5A, dtype=torch.uint8, device="cuda")
    sbuf = torch.full((rows + 2,), 7.25, dtype=torch.float32, device="cuda")
    N.check(L.cb_quantize_per_group_int8(x.data_ptr() + 2, N.CB_BF16, rows, G, 1e-12, qbuf.data_ptr() + pad + 1,
                                         sbuf.data_ptr() + 4, stream))
    torch.cuda.synchronize()
    assert (qbuf[:pad + 1] == 0x5A).all() and (qbuf[pad + 1 + rows * G:] == 0x5A).all()
    assert sbuf[0].item() == 7.25 and sbuf[-1].item() == 7.25
    q_ref, s_ref = O.int8_quantize_group(x[1:].cpu().view(rows, G), G)
    assert_bits_equal(qbuf[pad + 1:pad + 1 + rows * G].view(torch.int8).cpu(), q_ref.reshape(-1), "codes")
    assert_bits_equal(sbuf[1:-1], s_ref, "scales")


def test_split_phase_per_tensor_matches_single_call():
    """cb_amax_abs on two halves + max + cb_cast_per_tensor == the one-call result (the multi-GPU recipe)."""
    from cublade_b200 import _native as N
    from cublade_b200 import workloads as W

    L = N.lib()
    x = W.fp8_tensor_case(1024, 1024).cuda()
    n = x.numel()
    stream = torch.cuda.current_stream().cuda_stream
    parts = torch.zeros(2, dtype=torch.float32, device="cuda")
    half = n // 2
    N.check(L.cb_amax_abs(x.data_ptr(), N.CB_BF16, half, parts.data_ptr(), stream))
    N.check(L.cb_amax_abs(x.data_ptr() + 2 * half, N.CB_BF16, n - half, parts.data_ptr() + 4, stream))
    amax = parts.max().reshape(1)
    q = torch.empty(n, dtype=torch.uint8, device="cuda")
    s = torch.empty(1, dtype=torch.float32, device="cuda")
    N.check(L.cb_cast_per_tensor(x.data_ptr(), N.CB_BF16, n, amax.data_ptr(), 1e-12, N.CODE_E4M3, q.data_ptr(),
                                 s.data_ptr(), stream))
    q_ref, s_ref = O.fp8_quantize(x.cpu())
    assert_bits_equal(q.cpu(), q_ref.view(torch.uint8).reshape(-1), "codes")
    assert_bits_equal(s.reshape(()), s_ref, "scale")


def test_native_error_codes_and_python_exceptions():
    import cublade_b200 as cb
    from cublade_b200 import _native as N
    from cublade_b200.bindings.cuda import (dequantize_per_channel_int8, quantize_per_channel_int8,
                                            quantize_per_group_int8)

    x = torch.randn(4, 12, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="multiple of 16"):
        quantize_per_channel_int8(x)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        dequantize_per_channel_int8(torch.zeros(4, 12, dtype=torch.int8, device="cuda"),
                                    torch.ones(4, device="cuda"), torch.bfloat16)
    with pytest.raises(RuntimeError, match="group_size"):
        quantize_per_group_int8(torch.randn(2, 8192, device="cuda"), 8192)
    with pytest.raises(ValueError):
        cb.quantize_tensor(x.t(), dtype=torch.int8)  # not contiguous
    with pytest.raises(ValueError):
        cb.quantize_tensor(x.float(), dtype=torch.float8_e4m3fn)  # fp32 not accepted for FP8
    with pytest.raises(ValueError):
        cb.quantize_tensor(x, dtype=torch.float8_e4m3fn, mode="channel")
    with pytest.raises(ValueError):  # (any in-range axis is served; the reference raises NotImplementedError for != 0)
        cb.quantize_tensor(x, dtype=torch.int8, mode="channel", ch_axis=x.dim())
    with pytest.raises(NotImplementedError):
        cb.quantize_tensor(x, "asymmetric")
    with pytest.raises(ValueError, match="evenly divide"):
        cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=5, ch_axis=-1)
    qt = cb.quantize_tensor(x.float().contiguous(), dtype=torch.int8, mode="tensor")
    with pytest.raises(ValueError):  # quantized from fp32: no dequant path, as in the reference
        cb.dequantize_tensor(qt)
    # raw ABI: bad dtype code and null pointer are reported, nothing is launched
    assert N.lib().cb_quantize_per_tensor_fp8(x.data_ptr(), N.CB_F32, 8, 1e-12, x.data_ptr(), x.data_ptr(),
                                              x.data_ptr(), None) == 2
    assert N.lib().cb_dequantize_per_tensor_int8(None, None, 8, N.CB_BF16, None, None) == 1
    assert b"null" in N.lib().cb_last_error()
