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


# ------------------------------------------------------------------------------------------------
# per-GROUP along a non-last axis, quantized where the data lies (the reference copies the axis last
# and back: cublade/quantization/quantizers.py:122-132, dequantizers.py:58-72)
# ------------------------------------------------------------------------------------------------
GROUP_CASES = [
    # shape, axis, group size          kernel the launcher picks
    ((256, 64), 0, 32),              # vector: inner = 64
    ((4, 128, 24), 1, 32),           # vector, inner = 24 (3 bf16 packs)
    ((2, 96, 5, 8), 1, 16),          # vector, inner = 40
    ((3, 64, 6), 1, 64),             # scalar for 16-bit (inner = 6), one group per column
    ((8, 10, 7), 1, 5),              # scalar, odd sizes
    ((512, 128), 0, 128),            # vector, tall groups
    ((6, 4096, 16), 1, 4096),        # the largest group the reference accepts
    ((40, 12), 0, 1),                # group of one element
    ((2, 3, 64, 4), 2, 8),           # fp32 packs of 4 fit inner = 4; 16-bit scalar
    ((5, 32, 64), -2, 32),           # negative axis
]


@pytest.mark.parametrize("shape,axis,G", GROUP_CASES, ids=[f"{s}-ax{a}-g{g}" for s, a, g in GROUP_CASES])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_group_mode_along_a_non_last_axis_without_copies(shape, axis, G, dtype):
    import cublade_b200 as cb

    g = torch.Generator().manual_seed(abs(hash((shape, axis, G))) % (2 ** 31))
    x = (torch.randn(*shape, generator=g) * 1.3).to(dtype)
    idx = [slice(None)] * len(shape)
    idx[axis] = slice(0, G)
    x[tuple(idx)] *= 23.0                      # first group of every line: another range
    x.view(-1)[:: max(1, x.numel() // 7)] = 0  # some exact zeros
    if x.shape[axis] >= 2 * G:
        idx[axis] = slice(G, 2 * G)
        x[tuple(idx)] = 0                      # all-zero groups: scale = 1 / (127 / eps)
    ref = O.quantize_tensor(x, torch.int8, "group", group_size=G, ch_axis=axis)
    qt = cb.quantize_tensor(x.cuda(), dtype=torch.int8, mode="group", group_size=G, ch_axis=axis)
    assert qt.data.shape == x.shape and qt.data.is_contiguous() and qt.scale.shape == (x.numel() // G,)
    assert qt.axis == axis and qt.group_size == G
    assert_bits_equal(qt.scale, ref["scale"], "scales")
    assert_bits_equal(qt.data, ref["data"], "codes")
    if dtype == torch.float32:
        with pytest.raises(ValueError):
            cb.dequantize_tensor(qt)  # float32 origin cannot come back, as in the reference
        qt.original_dtype = ref["original_dtype"] = torch.float16
    assert_bits_equal(cb.dequantize_tensor(qt), O.dequantize_tensor(ref), "dequant")


def test_group_mode_non_last_axis_full_size_against_the_copying_route():
    """bf16 [8192, 8192] with groups of 128 down the rows (axis 0): codes, scales and dequantized values must equal
    what the library's contiguous-group kernels give on the transposed copy -- the route the reference takes."""
    import cublade_b200 as cb

    gen = torch.Generator(device="cuda").manual_seed(12)
    x = (torch.randn(8192, 8192, generator=gen, device="cuda") * 0.5).to(torch.bfloat16)
    qt = cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=128, ch_axis=0)
    moved = x.t().contiguous()
    want = cb.quantize_tensor(moved, dtype=torch.int8, mode="group", group_size=128, ch_axis=-1)
    assert torch.equal(qt.scale, want.scale)
    assert torch.equal(qt.data, want.data.t())
    assert torch.equal(cb.dequantize_tensor(qt), cb.dequantize_tensor(want).t())
    with pytest.raises(ValueError, match="evenly divide"):
        cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=96, ch_axis=0)
