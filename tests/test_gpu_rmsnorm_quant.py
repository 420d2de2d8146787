"""GPU parity of the fused RMSNorm -> per-row quantize kernel (called through the C ABI via its binding)
against the CPU formulation in oracle/oracle.py.

The op is announced by the reference (README.md:20) but not shipped, so the oracle is the unfused chain
"RMSNorm with an unfused layer's roundings, then the reference's per-channel quantizer".  The only number
whose last bits depend on the summation order is r = 1/rms per row: it is compared with the float64-sum
value to 2 float32 ulp; everything downstream (normalised rows, codes, scales) must then be bit-identical
to the oracle evaluated with the kernel's r.
"""
import pytest
import torch

from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _case(rows, hidden, dtype, seed, with_gain=True):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, hidden, generator=g) * 2.5).to(dtype)
    if hidden >= 16:
        x[:, 3] *= 20.0  # an outlier feature, as activations have
    gain = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype) if with_gain else None
    return x, gain


def _check(x, gain, code, rms_eps=1e-6):
    from cublade_b200.bindings.cuda import rmsnorm_quantize

    q, s, y, r = rmsnorm_quantize(x.cuda(), gain.cuda() if gain is not None else None, rms_eps=rms_eps, dtype=code,
                                  return_normed=True, return_rstd=True)
    assert q.shape == x.shape and q.dtype == code and s.shape == (x.shape[0],) and y.dtype == x.dtype
    _, _, _, r_exact = O.rmsnorm_quantize(x, gain, rms_eps, code)
    rel = ((r.cpu().double() - r_exact.double()).abs() / r_exact.double()).max().item()
    assert rel <= 2.5e-7, f"1/rms off by {rel:.2e} (more than 2 float32 ulp)"
    q_ref, s_ref, y_ref, _ = O.rmsnorm_quantize(x, gain, rms_eps, code, rstd=r)
    assert_bits_equal(y, y_ref, "normalised rows")
    assert_bits_equal(s, s_ref, "scales")
    assert_bits_equal(q, q_ref, "codes")


@pytest.mark.parametrize("hidden", [8, 64, 256, 512, 1024, 1032, 2048, 4096, 8192, 16384])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_register_resident_rows_int8(hidden, dtype):
    x, gain = _case(37, hidden, dtype, hidden)
    _check(x, gain, torch.int8)


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (300, 5120), (9, 100), (5, 16392), (3, 20000), (2, 7)])
@pytest.mark.parametrize("code", [torch.int8, torch.float8_e4m3fn])
def test_ragged_rows_long_rows_both_codes(rows, hidden, code):
    """Row lengths that are not a multiple of 8 or exceed 16 384 take the scalar kernel; both code kinds."""
    x, gain = _case(rows, hidden, torch.bfloat16, rows * 100003 + hidden)
    _check(x, gain, code)


def test_without_gain_zero_rows_and_tiny_rows():
    x, _ = _case(64, 2048, torch.bfloat16, 5, with_gain=False)
    x[7] = 0  # an all-zero token: r = 1/sqrt(eps), y = 0, scale = 1/(127/eps)
    x[9] *= 1e-18
    _check(x, None, torch.int8)
    _check(x, None, torch.float8_e4m3fn)


def test_container_api_round_trip_and_errors():
    import cublade_b200 as cb
    from cublade_b200.quantization import rmsnorm_quantize_tensor

    x, gain = _case(4 * 50, 4096, torch.bfloat16, 11)
    x3 = x.view(4, 50, 4096)
    qt = rmsnorm_quantize_tensor(x3.cuda(), gain.cuda())
    assert qt.mode == "channel" and qt.axis == 0 and qt.data.shape == (200, 4096) and qt.scale.shape == (200,)
    y_ref, _ = O.rmsnorm_rows(x, gain)
    y = cb.dequantize_tensor(qt).cpu().float()
    step = qt.scale.cpu()[:, None]
    # half a quantization step plus one bf16 ulp of the dequantized value
    assert ((y - y_ref.float()).abs() <= 0.5 * step + y_ref.float().abs() * 2.0 ** -7 + 1e-6).all()
    with pytest.raises(ValueError):
        rmsnorm_quantize_tensor(x3, gain)  # CPU tensor
    from cublade_b200.bindings.cuda import rmsnorm_quantize
    with pytest.raises(RuntimeError):
        rmsnorm_quantize(x.cuda().float())  # float32 activations are not served
    with pytest.raises(RuntimeError):
        rmsnorm_quantize(x.cuda(), gain.cuda().float())  # gain in another dtype


def test_full_size_against_unfused_chain_on_the_gpu():
    """16384 tokens x 8192 features: the fused kernel must equal the library's own per-channel quantizer
    applied to the normalised rows the kernel reports (same GPU arithmetic, two different kernels)."""
    from cublade_b200.bindings.cuda import quantize_per_channel_int8, rmsnorm_quantize

    g = torch.Generator(device="cuda").manual_seed(3)
    x = (torch.randn(16384, 8192, generator=g, device="cuda") * 1.7).to(torch.bfloat16)
    gain = (1.0 + 0.05 * torch.randn(8192, generator=g, device="cuda")).to(torch.bfloat16)
    q, s, y, r = rmsnorm_quantize(x, gain, return_normed=True, return_rstd=True)
    q2, s2 = quantize_per_channel_int8(y)
    assert torch.equal(q, q2) and torch.equal(s, s2)
    r_ref = torch.rsqrt(x.double().pow(2).mean(dim=1) + 1e-6)
    assert ((r.double() - r_ref).abs() / r_ref).max().item() <= 2.5e-7
    y_ref = ((x.float() * r[:, None]).to(torch.bfloat16).float() * gain.float()).to(torch.bfloat16)
    assert torch.equal(y.view(torch.int16), y_ref.view(torch.int16))
