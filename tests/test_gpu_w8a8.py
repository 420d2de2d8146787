"""GPU parity of the W8A8 linear (integer tensor cores, exact int32 accumulation) against the CPU
formulation in oracle.w8a8_forward.  The accumulation is exact and every floating-point step is a single
IEEE operation in a fixed order, so the comparison is bit for bit."""
import pytest
import torch

from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _problem(M, N, K, dtype, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    x = (torch.randn(M, K, generator=g) * 1.5).to(dtype)
    x[:, K // 3] *= 12.0  # an outlier feature
    b = torch.randn(N, generator=g).to(dtype) if bias else None
    return w, x, b, O.w8a16_quantize(w, dtype)


@pytest.mark.parametrize("M,N,K,bias", [(1, 64, 64, False), (3, 40, 128, True), (16, 256, 1024, True), (33, 130, 320, True),
                                        (70, 512, 4096, False), (256, 384, 512, True), (300, 1000, 2064, True),
                                        (5, 24, 72, True), (9, 17, 100, False)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_binding_matches_oracle_bit_for_bit(M, N, K, bias, dtype):
    """K % 16 == 0 runs on the tensor cores, the last two shapes on the plain kernel."""
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.w8a8 import w8a8_linear

    w, x, b, lay = _problem(M, N, K, dtype, M * 1000 + N + K, bias)
    xq, xs = O.int8_quantize_rows(x)
    y = w8a8_linear(xq.cuda(), xs.cuda(), lay["int8_weights"].cuda(), lay["scales"].cuda(), b.cuda() if bias else None,
                    out_dtype=dtype)
    want = O.w8a8_forward(x, lay, b, xq=xq, xs=xs)
    assert_bits_equal(y, want, "y")
    assert Nat.device_error_state() == 0


@pytest.mark.parametrize("M,N,K", [(512, 40000, 256), (300, 80000 + 128, 128), (1024, 24000, 192)])
def test_pair_kernel_with_several_tiles_per_cta_pair(M, N, K):
    """M >= 256 runs on pairs of CTAs (`tcgen05.mma.cta_group::2`): more 256-feature tiles than the 74 pairs of the
    GPU, so every pair walks through several tiles (ring and accumulator phases wrap, the hardware cluster barrier is
    reached once at the start and once at the end), with a ragged last tile in M and in N."""
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.w8a8 import w8a8_linear

    dtype = torch.bfloat16
    w, x, b, lay = _problem(M, N, K, dtype, M + N + K, True)
    xq, xs = O.int8_quantize_rows(x)
    y = w8a8_linear(xq.cuda(), xs.cuda(), lay["int8_weights"].cuda(), lay["scales"].cuda(), b.cuda(), out_dtype=dtype)
    assert_bits_equal(y, O.w8a8_forward(x, lay, b, xq=xq, xs=xs), "y")
    assert Nat.device_error_state() == 0


@pytest.mark.parametrize("M", [1, 16, 128, 2048])
def test_layer_config4_shapes_and_accuracy(M):
    """N = 14336, K = 4096 (the W8A16 benchmark shape).  The layer must equal the oracle bit for bit and stay
    close to the unquantized product."""
    import cublade_b200 as cb
    from cublade_b200 import workloads as W

    w, x, _ = W.w8a16_case(M)
    layer = cb.quantization.cuBladeW8A8LinearLayer(4096, 14336, bias=False, dtype=torch.bfloat16)
    layer.quantize(w)
    layer = layer.cuda()
    ref_layer = O.w8a16_quantize(w, torch.bfloat16)
    assert_bits_equal(layer.int8_weights, ref_layer["int8_weights"], "int8 weights")
    y = layer(x.cuda())
    assert y.shape == (M, 14336) and y.dtype == torch.bfloat16
    assert_bits_equal(y, O.w8a8_forward(x, ref_layer), "y")
    if M <= 128:
        exact = x.double() @ w.double().t()
        rel = ((y.cpu().double() - exact).norm() / exact.norm()).item()
        assert rel < 3e-2, f"relative Frobenius error vs the unquantized product {rel:.3e}"


def test_quantize_model_w8a8_and_fused_rmsnorm_input():
    import torch.nn as nn

    import cublade_b200 as cb
    from cublade_b200.quantization import rmsnorm_quantize_tensor

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 512), nn.ReLU(), nn.Linear(512, 64)).to(torch.bfloat16)
    x = torch.randn(40, 256).to(torch.bfloat16)
    want = model(x).float()
    qmodel = cb.quantize_model(model, "w8a8", inplace=False).cuda()
    assert all(isinstance(m, cb.quantization.cuBladeW8A8LinearLayer) for m in (qmodel[0], qmodel[2]))
    got = qmodel(x.cuda()).cpu().float()
    assert ((got - want) ** 2).mean().item() < 1e-2 and (got - want).abs().max().item() < 0.5
    # a per-token QuantizedTensor (here from the fused RMSNorm) feeds the layer without a second quantization pass
    gain = torch.ones(256, dtype=torch.bfloat16)
    qt = rmsnorm_quantize_tensor(x.cuda(), gain.cuda())
    y = qmodel[0](qt)
    lay = {"int8_weights": qmodel[0].int8_weights.cpu(), "scales": qmodel[0].scales.cpu()}
    want_y = O.w8a8_forward(x, lay, qmodel[0].bias.detach().cpu(), xq=qt.data.cpu(), xs=qt.scale.cpu())
    assert_bits_equal(y, want_y, "layer on a fused-RMSNorm input")
    with pytest.raises(ValueError):
        qmodel[0](x)  # CPU tensor
