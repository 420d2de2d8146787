"""GPU parity of per-channel INT8 along any axis (quantized in place, no transpose) against the CPU
formulation "move the axis to the front, run the reference's axis-0 quantizer, move it back"
(oracle.int8_quantize_axis, following cublade/kernels/cuda/quantization/quantize_int8.cu:487-509).
Bit-exact: codes, scales, dequantized values."""
import pytest
import torch

from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402

CASES = [
    # shape, axis                      layout the launcher picks
    ((64, 96, 3, 8), 1),             # runs: inner = 24 (bf16 packs of 8 inside a run)
    ((5, 16, 40), 1),                # runs, 40 = 5 packs
    ((300, 4096), 1),                # last axis, C % 8 == 0
    ((300, 4096), -1),
    ((7, 33, 2048), 2),              # last axis with an outer product of two axes
    ((4, 10, 6), 1),                 # inner = 6: scalar
    ((9, 1001), 1),                  # last axis, C % 8 != 0: scalar
    ((3, 5, 7, 11), 2),              # scalar
    ((128, 256), 0),                 # axis 0 through the per-axis entry point: outer = 1
    ((1, 512, 16), 1),
    ((2, 1, 64), 1),                 # one channel
]


@pytest.mark.parametrize("shape,axis", CASES, ids=[f"{s}-ax{a}" for s, a in CASES])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quantize_and_dequantize_any_axis(shape, axis, dtype):
    from cublade_b200.bindings.cuda import dequantize_per_axis_int8, quantize_per_axis_int8

    g = torch.Generator().manual_seed(abs(hash((shape, axis))) % (2 ** 31))
    x = (torch.randn(*shape, generator=g) * 1.3).to(dtype)
    idx = [slice(None)] * len(shape)
    idx[axis] = 0
    x[tuple(idx)] *= 37.0  # channels with very different ranges
    if x.shape[axis] > 1:
        idx[axis] = 1
        x[tuple(idx)] = 0  # an all-zero channel: scale = 1 / (127 / eps)
    q, s = quantize_per_axis_int8(x.cuda(), axis)
    q_ref, s_ref = O.int8_quantize_axis(x, axis)
    assert q.shape == x.shape and s.shape == (x.shape[axis],)
    assert_bits_equal(s, s_ref, "scales")
    assert_bits_equal(q, q_ref, "codes")
    for dt in (torch.bfloat16, torch.float16):
        y = dequantize_per_axis_int8(q, s, axis, dt)
        assert_bits_equal(y, O.int8_dequantize_axis(q_ref, s_ref, axis % len(shape), dt), f"dequant {dt}")


def test_quantize_tensor_routes_other_axes_and_round_trips():
    import cublade_b200 as cb

    g = torch.Generator().manual_seed(5)
    x = (torch.randn(2048, 1024, generator=g) * torch.logspace(-2, 2, 1024)[None, :]).to(torch.bfloat16)
    qt = cb.quantize_tensor(x.cuda(), dtype=torch.int8, mode="channel", ch_axis=1)
    assert qt.axis == 1 and qt.scale.shape == (1024,)
    q_ref, s_ref = O.int8_quantize_axis(x, 1)
    assert_bits_equal(qt.data, q_ref, "codes")
    assert_bits_equal(qt.scale, s_ref, "scales")
    y = cb.dequantize_tensor(qt)
    assert_bits_equal(y, O.int8_dequantize_axis(q_ref, s_ref, 1, torch.bfloat16), "dequant")
    # per-column scales keep every column within half a step; one scale per row could not
    err = (y.cpu().float() - x.float()).abs()
    assert (err <= 0.5 * s_ref[None, :] * 1.01 + x.float().abs() * 2.0 ** -8 + 1e-30).all()  # + bf16 rounding of y


def test_full_size_last_axis_equals_transposed_axis0_path_on_the_gpu():
    """8192 x 8192 bf16 quantized per COLUMN in place must equal the library's axis-0 kernel run on the
    transposed copy (two different kernels, same arithmetic), and survive a dequantize round trip."""
    from cublade_b200.bindings.cuda import dequantize_per_axis_int8, quantize_per_axis_int8, quantize_per_channel_int8

    g = torch.Generator(device="cuda").manual_seed(9)
    x = (torch.randn(8192, 8192, generator=g, device="cuda") * 0.7).to(torch.bfloat16)
    q, s = quantize_per_axis_int8(x, 1)
    qt, st = quantize_per_channel_int8(x.t().contiguous())
    assert torch.equal(s, st) and torch.equal(q, qt.t())
    y = dequantize_per_axis_int8(q, s, 1)
    assert ((y.float() - x.float()).abs() <= 0.5 * s[None, :] + x.float().abs() * 2.0 ** -8 + 1e-30).all()
