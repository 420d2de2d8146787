"""GPU parity of the W4A16 path against the CPU formulation in oracle/: the 4-bit row quantizer and the
unpacker bit for bit, the linear within the W8A16 tolerance (relative Frobenius error <= 1e-2 and max abs
error <= 2e-2 * max|ref| against the reference's rounding order, oracle.w8a16_forward on the 4-bit codes)."""
import io

import pytest
import torch

from tests.helpers import assert_bits_equal, max_abs_ratio, rel_fro

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402

REL_FRO_TOL = 1e-2
MAX_ABS_TOL = 2e-2


def _check(y, ref, what):
    rf, ma = rel_fro(y, ref), max_abs_ratio(y, ref)
    assert rf <= REL_FRO_TOL and ma <= MAX_ABS_TOL, f"{what}: rel_fro={rf:.3e} max_abs_ratio={ma:.3e}"


@pytest.mark.parametrize("N,K", [(1, 8), (16, 64), (33, 200), (256, 4096), (7, 8192)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_quantizer_and_unpacker_bit_exact(N, K, dtype):
    from cublade_b200.bindings.w4a16 import w4_quantize_rows, w4_unpack

    g = torch.Generator().manual_seed(N * 131 + K)
    w = (torch.randn(N, K, generator=g) * 0.03).to(dtype)
    w[0, : min(K, 8)] = 0.0
    if N > 2:
        w[2] = 0.0  # an all-zero row: amax clamps to eps, codes 0
        w[1, K // 2] = 0.9  # a dominant element
    packed, scale = w4_quantize_rows(w.cuda())
    q_ref, s_ref = O.int4_quantize_rows(w)
    assert_bits_equal(scale, s_ref, "scale")
    assert_bits_equal(packed, O.int4_pack(q_ref), "packed codes")
    assert_bits_equal(w4_unpack(packed), q_ref, "unpacked codes")


def test_unpack_every_nibble_value():
    from cublade_b200.bindings.w4a16 import w4_unpack

    codes = torch.arange(-8, 8, dtype=torch.int8).repeat(4, 3)  # [4, 48], every value in every byte position
    codes = torch.stack([codes[0], codes[1].roll(1), codes[2].roll(3), codes[3].roll(5)])
    assert_bits_equal(w4_unpack(O.int4_pack(codes).cuda()), codes, "codes")


def _problem(M, N, K, dtype, seed, bias):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    x = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(N, generator=g).to(dtype) if bias else None
    return w, x, b, O.w4a16_quantize(w, dtype)


# M <= 16 with K % 128 == 0 and N % 16 == 0 streams the packed weights; the rest unpacks and runs the W8A16 path
@pytest.mark.parametrize("M,N,K,bias", [(1, 16, 128, False), (2, 32, 64, True), (1, 512, 4096, True), (5, 64, 1024, True), (8, 256, 2048, False),
                                        (9, 128, 1088, True), (16, 512, 4096, True), (17, 256, 1024, True),
                                        (64, 384, 2048, False), (300, 512, 1024, True), (4, 24, 72, True), (3, 40, 8, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_linear_matches_oracle(M, N, K, bias, dtype):
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.w4a16 import w4a16_linear

    w, x, b, lay = _problem(M, N, K, dtype, M * 1000 + N + K, bias)
    y = w4a16_linear(x.cuda(), lay["int4_weights"].cuda(), lay["scales"].cuda(), b.cuda() if bias else None)
    assert y.shape == (M, N) and y.dtype == dtype
    _check(y, O.w8a16_forward(x, lay, b), f"M={M} N={N} K={K}")
    assert Nat.device_error_state() == 0


def test_strided_activations_and_argument_errors():
    from cublade_b200.bindings.w4a16 import w4a16_linear

    w, x, b, lay = _problem(6, 64, 256, torch.bfloat16, 5, True)
    wide = torch.zeros(6, 300, dtype=torch.bfloat16)
    wide[:, :256] = x
    y = w4a16_linear(wide.cuda()[:, :256], lay["int4_weights"].cuda(), lay["scales"].cuda(), b.cuda())
    _check(y, O.w8a16_forward(x, lay, b), "strided rows")
    with pytest.raises(ValueError):
        w4a16_linear(x, lay["int4_weights"].cuda(), lay["scales"].cuda())  # CPU activations
    with pytest.raises(ValueError):
        w4a16_linear(x.cuda()[:, :128], lay["int4_weights"].cuda(), lay["scales"].cuda())  # K mismatch
    with pytest.raises(NotImplementedError):
        w4a16_linear(x.float().cuda(), lay["int4_weights"].cuda(), lay["scales"].cuda())


def test_layer_quantize_model_and_checkpoint():
    import cublade_b200 as cb
    from cublade_b200.quantization.checkpoint import load_quantized_model, save_quantized_model

    torch.manual_seed(11)
    model = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 64)).to(torch.bfloat16)
    ref_w = [model[0].weight.detach().clone(), model[2].weight.detach().clone()]
    ref_b = [model[0].bias.detach().clone(), model[2].bias.detach().clone()]
    qmodel = cb.quantize_model(model, "w4a16", inplace=False).cuda()
    assert isinstance(qmodel[0], cb.quantization.cuBladeW4A16LinearLayer)
    lay0 = O.w4a16_quantize(ref_w[0], torch.bfloat16)
    assert_bits_equal(qmodel[0].int4_weights, lay0["int4_weights"], "layer 0 packed weights")
    assert_bits_equal(qmodel[0].scales, lay0["scales"], "layer 0 scales")
    x = torch.randn(3, 5, 256).to(torch.bfloat16)
    y = qmodel(x.cuda())
    h = torch.nn.functional.gelu(O.w8a16_forward(x, lay0, ref_b[0]).float()).to(torch.bfloat16)
    want = O.w8a16_forward(h, O.w4a16_quantize(ref_w[1], torch.bfloat16), ref_b[1])
    assert y.shape == (3, 5, 64)
    assert rel_fro(y, want) <= 2e-2
    buf = io.BytesIO()
    save_quantized_model(qmodel, buf)
    buf.seek(0)
    fresh = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 64)).to(torch.bfloat16)
    loaded = load_quantized_model(fresh, buf).cuda()
    assert_bits_equal(loaded(x.cuda()), y, "forward after the checkpoint round trip")
