"""Seeded random-shape parity sweeps on the GPU: the public quantize / dequantize API bit for bit against the CPU
oracle over shapes, axes, group sizes, dtypes and value distributions nobody picked by hand, and the W8A16 linear
(every kernel path, with and without bias / outlier columns) within the stated tolerance of a float64 evaluation
of the reference's formula (cublade/quantization/quantizers.py:101-139, dequantizers.py:38-75, linear.py:97-135).
The hand-written cases of the other files pin the corners; these catch what lies between them."""
import random

import pytest
import torch

from tests.helpers import assert_bits_equal, max_abs_ratio, rel_fro

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _values(shape, dtype, rng, g):
    """Normal data with one of several twists: a few huge entries, an all-zero slice, a constant tensor, tiny values."""
    x = torch.randn(*shape, generator=g) * rng.choice([1e-3, 0.3, 1.0, 40.0])
    twist = rng.randrange(5)
    flat = x.view(-1)
    if twist == 0 and flat.numel() > 4:
        idx = torch.randint(0, flat.numel(), (4,), generator=g)
        flat[idx] = flat[idx] * 300.0
    elif twist == 1:
        x[..., 0] = 0.0
    elif twist == 2:
        x.fill_(rng.choice([0.0, 1.0, -2.5]))
    elif twist == 3:
        x = x * 1e-30
    return x.to(dtype)


def _quant_cases(n, seed):
    rng = random.Random(seed)
    cases = []
    for i in range(n):
        nd = rng.choice([1, 2, 2, 2, 3, 4])
        mode = rng.choice(["tensor", "tensor_fp8", "channel", "group", "group"])
        dtype = rng.choice([torch.bfloat16, torch.float16, torch.float32])
        if mode == "tensor_fp8" and dtype == torch.float32:
            dtype = torch.bfloat16
        if mode in ("channel", "group") and nd == 1:
            nd = 2
        shape = [rng.choice([1, 2, 3, 5, 8, 16, 24, 33, 64, 100, 128, 256, 520]) for _ in range(nd)]
        axis, group = 0, 32
        if mode == "channel":
            # the reference's kernel needs rows of a multiple of 16 bytes (other lengths raise there and here)
            lanes = 16 // torch.empty((), dtype=dtype).element_size()
            shape[-1] = -(-shape[-1] // lanes) * lanes
        if mode == "group":
            axis = rng.randrange(nd)
            group = rng.choice([8, 16, 32, 64, 128])
            shape[axis] = group * rng.choice([1, 2, 3, 5])
        cases.append((i, tuple(shape), mode, axis, group, dtype))
    return cases


QUANT_CASES = _quant_cases(120, seed=20240611)


@pytest.mark.parametrize("case", QUANT_CASES, ids=[f"{c[0]}-{c[2]}-{'x'.join(map(str, c[1]))}-ax{c[3]}-g{c[4]}-{str(c[5])[6:]}"
                                                    for c in QUANT_CASES])
def test_quantize_tensor_and_back_equal_the_oracle(case):
    import cublade_b200 as cb

    i, shape, mode, axis, group, dtype = case
    rng = random.Random(1000 + i)
    g = torch.Generator().manual_seed(1000 + i)
    x = _values(shape, dtype, rng, g)
    kw = dict(dtype=torch.float8_e4m3fn, mode="tensor") if mode == "tensor_fp8" else \
        dict(dtype=torch.int8, mode=mode, group_size=group, ch_axis=axis)
    want = O.quantize_tensor(x, **kw)
    got = cb.quantize_tensor(x.cuda(), **kw)
    assert got.mode == want["mode"] and got.axis == want["axis"] and got.original_dtype == dtype
    assert_bits_equal(got.scale.reshape(-1), want["scale"].reshape(-1), "scales")
    assert_bits_equal(got.data, want["data"], "codes")
    if dtype == torch.float32:
        with pytest.raises(ValueError):  # as the reference: a tensor quantized from float32 cannot come back
            cb.dequantize_tensor(got)
        return
    assert_bits_equal(cb.dequantize_tensor(got), O.dequantize_tensor(want), "dequantized")


def _linear_cases(n, seed):
    rng = random.Random(seed)
    cases = []
    for i in range(n):
        cases.append((i,
                      rng.choice([1, 2, 7, 8, 9, 16, 17, 31, 64, 65, 128, 129, 200, 208, 209, 300, 416, 500, 833]),  # M
                      rng.choice([8, 16, 24, 120, 128, 136, 256, 512, 1000, 1024, 2040]),                          # N
                      rng.choice([16, 32, 64, 72, 80, 128, 200, 320, 448, 1024, 2048]),                            # K
                      rng.choice([0, 0, 0, 1, 3, 8, 16, 24, 72]),                                                   # KO
                      rng.choice([torch.bfloat16, torch.float16]), rng.random() < 0.5, rng.choice([0, 0, 1, 3, 2])))
    return cases


LINEAR_CASES = _linear_cases(90, seed=77)


@pytest.mark.parametrize("case", LINEAR_CASES,
                         ids=[f"{c[0]}-M{c[1]}-N{c[2]}-K{c[3]}-KO{c[4]}-{str(c[5])[6:]}-b{int(c[6])}-p{c[7]}" for c in LINEAR_CASES])
def test_w8a16_linear_every_path_against_float64(case):
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.w8a16 import w8a16_linear

    i, M, N, K, KO, dtype, with_bias, path = case
    g = torch.Generator().manual_seed(5000 + i)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    x = torch.randn(M, K, generator=g).to(dtype)
    bias = torch.randn(N, generator=g).to(dtype) if with_bias else None
    lay = O.w8a16_quantize(w, dtype)
    ref = O.w8a16_forward_fp64(x, lay, bias)
    xo = wo = None
    if KO:
        xo = (torch.randn(M, KO, generator=g) * 4).to(dtype)
        wo = (torch.randn(N, KO, generator=g) * 0.05).to(dtype)
        ref = ref + xo.double() @ wo.double().T
    try:
        y = w8a16_linear(x.cuda(), lay["int8_weights"].cuda(), lay["scales"].cuda(), bias.cuda() if with_bias else None,
                         xo.cuda() if KO else None, wo.cuda() if KO else None, path=path)
    except NotImplementedError:
        assert path in (2, 3)  # a forced tensor-core path may refuse a shape; the automatic one never does
        pytest.skip("shape not served by the forced path")
    torch.cuda.synchronize()
    assert Nat.device_error_state() == 0
    assert torch.isfinite(y).all()
    # the tolerance stated for the layer: relative Frobenius 1e-2, largest deviation 2e-2 of the largest value
    assert rel_fro(y, ref) <= 1e-2
    assert max_abs_ratio(y, ref) <= 2e-2


def _w8a8_cases(n, seed):
    rng = random.Random(seed)
    return [(i, rng.choice([1, 2, 9, 16, 31, 64, 100, 255, 256, 300, 513]), rng.choice([8, 17, 40, 128, 130, 384, 1000, 2050]),
             rng.choice([16, 64, 72, 100, 128, 320, 1024, 2064]), rng.choice([torch.bfloat16, torch.float16]), rng.random() < 0.5)
            for i in range(n)]


W8A8_CASES = _w8a8_cases(40, seed=5)


@pytest.mark.parametrize("case", W8A8_CASES, ids=[f"{c[0]}-M{c[1]}-N{c[2]}-K{c[3]}-{str(c[4])[6:]}-b{int(c[5])}" for c in W8A8_CASES])
def test_w8a8_linear_bit_for_bit(case):
    """Integer tensor cores with exact int32 accumulation: equal to the CPU formulation bit for bit at every shape."""
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.w8a8 import w8a8_linear

    i, M, N, K, dtype, with_bias = case
    g = torch.Generator().manual_seed(9000 + i)
    w = (torch.randn(N, K, generator=g) * 0.05).to(dtype)
    x = (torch.randn(M, K, generator=g) * 1.5).to(dtype)
    b = torch.randn(N, generator=g).to(dtype) if with_bias else None
    lay = O.w8a16_quantize(w, dtype)
    xq, xs = O.int8_quantize_rows(x)
    y = w8a8_linear(xq.cuda(), xs.cuda(), lay["int8_weights"].cuda(), lay["scales"].cuda(), b.cuda() if with_bias else None,
                    out_dtype=dtype)
    assert_bits_equal(y, O.w8a8_forward(x, lay, b, xq=xq, xs=xs), "y")
    assert Nat.device_error_state() == 0


def _gemm_cases(n, seed):
    rng = random.Random(seed)
    return [(i, rng.choice([1, 5, 16, 64, 100, 128, 257, 512, 1000]), rng.choice([1, 7, 16, 96, 128, 200, 520, 1024]),
             rng.choice([1, 9, 16, 64, 100, 128, 1000, 2048]), rng.choice([torch.bfloat16, torch.float16, torch.int8]),
             rng.choice(["", "leaky_relu"])) for i in range(n)]


GEMM_CASES = _gemm_cases(40, seed=6)


@pytest.mark.parametrize("case", GEMM_CASES, ids=[f"{c[0]}-M{c[1]}-N{c[2]}-K{c[3]}-{str(c[4])[6:]}-{c[5] or 'none'}" for c in GEMM_CASES])
def test_generic_matmul_random_shapes(case):
    """matmul(A, B, activation) (cublade/bindings/triton/matmul.py:17-132) on the tcgen05 GEMM: int8 exact, 16-bit within
    one rounding of a float64 product."""
    from cublade_b200 import _native as Nat
    from cublade_b200.bindings.triton import matmul

    i, M, N, K, dtype, activation = case
    g = torch.Generator().manual_seed(12000 + i)
    if dtype == torch.int8:
        a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
        b = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int8)
        got = matmul(a.cuda(), b.cuda(), activation=activation).cpu()
        assert got.dtype == torch.int32 and torch.equal(got, (a.double() @ b.double()).to(torch.int32))
    else:
        a = torch.randn(M, K, generator=g).to(dtype)
        b = torch.randn(K, N, generator=g).to(dtype)
        ref = a.double() @ b.double()
        if activation == "leaky_relu":
            ref = torch.where(ref >= 0, ref, 0.01 * ref)
        got = matmul(a.cuda(), b.cuda(), activation=activation).cpu()
        assert got.dtype == dtype and got.shape == (M, N)
        assert rel_fro(got, ref) < (3e-3 if dtype == torch.bfloat16 else 5e-4)
    assert Nat.device_error_state() == 0
