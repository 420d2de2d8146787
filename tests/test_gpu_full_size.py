"""Full-size runs of the benchmark configurations that are too large to push through the CPU oracle
whole.  Parity is checked through properties that do not depend on size -- the emitted scale equals
the kernel formula applied to an independently computed amax, every element satisfies the round-trip
error bound -- and bit for bit against the oracle on random slices of the same tensors."""
import pytest
import torch

from tests.helpers import assert_bits_equal

pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


def _free_gib():
    free, _ = torch.cuda.mem_get_info()
    return free / 2**30


def test_config3_int8_per_group_full_size_properties_and_slices():
    import cublade_b200 as cb
    from cublade_b200 import workloads as W

    if _free_gib() < 8:
        pytest.skip("needs ~4 GiB of device memory")
    x_cpu = W.int8_group_case()  # 16384 x 8192, Student-t(3) * 0.5, seed 2
    x = x_cpu.cuda()
    qt = cb.quantize_tensor(x, dtype=torch.int8, mode="group", group_size=128, ch_axis=-1)
    assert qt.scale.shape == (x.numel() // 128,) and qt.data.shape == x.shape
    # scale = 1 / (127 / max(amax, eps)) with amax computed by torch on the device (IEEE fp32 division)
    amax = x.float().view(-1, 128).abs().amax(dim=1).clamp_min(1e-12)
    inv = torch.tensor(127.0, device="cuda") / amax
    assert torch.equal(qt.scale, torch.tensor(1.0, device="cuda") / inv)
    # |q| <= 127 and the group maximum maps to +-127
    q = qt.data.view(-1, 128)
    assert int(q.abs().max()) <= 127
    assert bool((q.abs().amax(dim=1) == 127).all())
    # round trip: |y - x| <= scale/2 (rounding to the code grid) + 2^-8 |y| (bf16 rounding of the product)
    for out_dtype in (torch.bfloat16, torch.float16):
        qt.original_dtype = out_dtype
        y = cb.dequantize_tensor(qt).float().view(-1, 128)
        err = (y - x.float().view(-1, 128)).abs()
        bound = qt.scale[:, None] * 0.5 * (1 + 2**-20) + y.abs() * 2**-8 + 1e-30
        assert bool((err <= bound).all()), f"round-trip bound violated for {out_dtype}"
    # bit-exact against the oracle on ALL 16384 rows, 2048 rows at a time
    q_all, s_all = qt.data.cpu(), qt.scale.cpu().view(x.shape[0], -1)
    for r0 in range(0, x.shape[0], 2048):
        q_ref, s_ref = O.int8_quantize_group(x_cpu[r0:r0 + 2048].reshape(-1, 128), 128)
        assert_bits_equal(q_all[r0:r0 + 2048].reshape(-1, 128), q_ref, f"codes of rows {r0}..")
        assert_bits_equal(s_all[r0:r0 + 2048].reshape(-1), s_ref, f"scales of rows {r0}..")


def test_config5_fp8_per_tensor_2_pow_33_elements():
    """The sharded FP8 configuration on one GPU: 2^33 bf16 elements (16 GiB in, 8 GiB codes, 16 GiB out)."""
    from cublade_b200 import workloads as W
    from cublade_b200.bindings.cuda import dequantize_per_tensor_fp8
    from cublade_b200.sharding import quantize_tensor_sharded

    if _free_gib() < 60:
        pytest.skip("needs ~42 GiB of device memory")
    chunk, nchunks = 1 << 27, 64
    x = torch.empty(chunk * nchunks, dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros((), device="cuda")
    for c in range(nchunks):
        part = W.sharded_fp8_chunk(c, chunk)
        x[c * chunk:(c + 1) * chunk] = part
        amax = torch.maximum(amax, part.float().abs().max())
    qt = quantize_tensor_sharded(x, dtype=torch.float8_e4m3fn)  # world size 1: no collective
    inv = torch.tensor(448.0, device="cuda") / amax.clamp_min(1e-12)
    assert torch.equal(qt.scale, torch.tensor(1.0, device="cuda") / inv)
    assert qt.data.numel() == 1 << 33
    # bit-exact against the oracle's arithmetic on four 1 Mi-element slices, using the global amax
    inv_cpu = inv.cpu()
    for c in (0, 17, 40, 63):
        lo = c * chunk + 12345
        xs = x[lo:lo + (1 << 20)].cpu()
        want = (xs.float() * inv_cpu).to(torch.float8_e4m3fn)
        assert_bits_equal(qt.data[lo:lo + (1 << 20)], want, f"codes of slice in chunk {c}")
    # dequantize and bound the round-trip error chunk by chunk: E4M3 keeps 3 mantissa bits
    # (relative step 2^-3 -> error <= 2^-4 |v|, or half the subnormal step 2^-10 in code units), plus bf16 rounding
    y = dequantize_per_tensor_fp8(qt.data, qt.scale, torch.bfloat16)
    s = qt.scale.item()
    for c in range(0, nchunks, 9):
        xs = x[c * chunk:(c + 1) * chunk].float()
        ys = y[c * chunk:(c + 1) * chunk].float()
        bound = xs.abs() * (2**-4 + 2**-8) + s * 2**-10 * 1.01
        assert bool(((ys - xs).abs() <= bound).all()), f"round-trip bound violated in chunk {c}"
    del x, y, qt
    torch.cuda.empty_cache()
