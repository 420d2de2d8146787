"""GPU parity of ``wmma_gemm`` (tcgen05 replacement for the reference's WMMA GEMM, cublade/kernels/cuda/wmma.cu)
against CPU matrix products.  8-bit inputs accumulate exactly in int32: bit for bit.  16-bit inputs accumulate in
fp32 in an order the hardware chooses: relative Frobenius error <= 1e-5 against a float64 product (the
reference's own demo compares with torch.matmul to 1e-2, examples/kernels/wmma_gemm.py)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(16, 16, 16), (128, 256, 64), (256, 512, 4096), (300, 1000, 2064), (33, 130, 320), (1024, 1024, 1024),
          (5, 24, 72), (9, 17, 100)]  # the last two: K * element size not a multiple of 16 -> plain kernel


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("dtype", [torch.int8, torch.uint8])
def test_integer_inputs_are_exact(M, N, K, dtype):
    from cublade_b200.bindings.cuda import wmma_gemm

    g = torch.Generator().manual_seed(M + N + K)
    lo, hi = (-128, 128) if dtype == torch.int8 else (0, 256)
    a = torch.randint(lo, hi, (M, K), generator=g).to(dtype)
    b = torch.randint(lo, hi, (K, N), generator=g).to(dtype)
    c = wmma_gemm(a.cuda(), b.cuda())
    want = (a.double() @ b.double()).to(torch.int32)  # exact in float64
    assert c.dtype == torch.int32 and c.shape == (M, N)
    assert torch.equal(c.cpu(), want)


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("dtype,acc", [(torch.float16, None), (torch.float16, torch.float16), (torch.bfloat16, None)])
def test_float_inputs_within_tolerance(M, N, K, dtype, acc):
    from cublade_b200.bindings.cuda import wmma_gemm

    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g).to(dtype)
    b = (torch.randn(K, N, generator=g) / K ** 0.5).to(dtype)
    c = wmma_gemm(a.cuda(), b.cuda(), acc)
    want = a.double() @ b.double()
    assert c.dtype == (acc or torch.float32)
    rel = ((c.cpu().double() - want).norm() / want.norm()).item()
    assert rel <= (1e-3 if acc == torch.float16 else 1e-5), f"relative Frobenius error {rel:.2e}"


def test_argument_checks_follow_the_reference():
    from cublade_b200 import _native as N
    from cublade_b200.bindings.cuda import wmma_gemm

    a = torch.randn(32, 32, device="cuda").half()
    with pytest.raises(RuntimeError, match="CUDA"):
        wmma_gemm(a.cpu(), a.cpu())
    with pytest.raises(RuntimeError, match="2D"):
        wmma_gemm(a[None], a)
    with pytest.raises(RuntimeError, match="incompatible"):
        wmma_gemm(a, a[:16])
    with pytest.raises(RuntimeError, match="same dtype"):
        wmma_gemm(a, a.bfloat16())
    with pytest.raises(RuntimeError, match="Unsupported dtype"):
        wmma_gemm(a.float(), a.float())
    with pytest.raises(RuntimeError, match="bfloat16"):
        wmma_gemm(a.bfloat16(), a.bfloat16(), torch.float16)
    with pytest.raises(RuntimeError, match="int32"):
        wmma_gemm(a.to(torch.int8), a.to(torch.int8), torch.float32)
    assert N.device_error_state() == 0


@pytest.mark.parametrize("M,N,K", [(64, 96, 128), (300, 520, 1000), (2048, 1024, 4096), (5, 7, 9)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.int8])
@pytest.mark.parametrize("activation", ["", "leaky_relu"])
def test_generic_matmul_wrapper(M, N, K, dtype, activation):
    """matmul(A, B, activation) with the contract of cublade/bindings/triton/matmul.py:17-132: C in the input dtype
    (int32 for int8), leaky_relu applied to the fp32 accumulator before the one rounding, ignored for int8."""
    from cublade_b200.bindings.triton import matmul

    g = torch.Generator().manual_seed(M + N + K)
    if dtype == torch.int8:
        a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8)
        b = torch.randint(-128, 128, (K, N), generator=g, dtype=torch.int8)
        want = (a.double() @ b.double()).to(torch.int32)
        got = matmul(a.cuda(), b.cuda(), activation=activation).cpu()
        assert got.dtype == torch.int32 and torch.equal(got, want)
        return
    a = torch.randn(M, K, generator=g).to(dtype)
    b = torch.randn(K, N, generator=g).to(dtype)
    ref = a.double() @ b.double()
    if activation == "leaky_relu":
        ref = torch.where(ref >= 0, ref, 0.01 * ref)
    got = matmul(a.cuda(), b.cuda(), activation=activation, override_config={"BLOCK_M": 64}, use_autotune=False).cpu()
    assert got.dtype == dtype and got.shape == (M, N)
    err = (got.double() - ref).norm() / ref.norm()
    assert err < (3e-3 if dtype == torch.bfloat16 else 5e-4), err  # one rounding to the 16-bit type
    with pytest.raises(ValueError, match="Unsupported dtype"):
        matmul(a.float().cuda(), b.float().cuda())
