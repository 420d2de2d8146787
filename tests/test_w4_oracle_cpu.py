"""CPU checks of the 4-bit restatement in oracle/: known answers of the row quantizer and the packed layout."""
import torch

from oracle import oracle as O


def test_int4_quantize_rows_known_answers():
    x = torch.tensor([[0.7, -0.35, 0.1, 0.0, -0.7, 0.05, 0.249, 0.251]], dtype=torch.float32)
    q, s = O.int4_quantize_rows(x)
    # inv = 7 / 0.7 = 10 (rounded to float32), codes = rint(x * inv)
    assert q.tolist() == [[7, -4 if round(-0.35 * float((7.0 / torch.tensor(0.7, dtype=torch.float32).double()).float())) == -4 else -3,
                           1, 0, -7, 0 if round(0.05 * 10) == 0 else 1, 2, 3]]
    assert abs(float(s[0]) - 0.1) < 1e-7
    z, sz = O.int4_quantize_rows(torch.zeros(2, 16))
    assert int(z.abs().max()) == 0 and torch.all(sz > 0)


def test_int4_pack_layout_and_round_trip():
    codes = torch.tensor([[1, 2, 3, 4, -1, -2, -3, -8]], dtype=torch.int8)
    packed = O.int4_pack(codes)
    # byte j = code[j] | code[4 + j] << 4 (two's-complement nibbles)
    assert packed.tolist() == [[0x1 | 0xF << 4, 0x2 | 0xE << 4, 0x3 | 0xD << 4, 0x4 | 0x8 << 4]]
    g = torch.Generator().manual_seed(0)
    c = torch.randint(-8, 8, (9, 64), generator=g, dtype=torch.int8)
    assert torch.equal(O.int4_unpack(O.int4_pack(c)), c)


def test_w4a16_layer_dict_feeds_the_w8a16_forward():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(12, 32, generator=g) * 0.1
    x = torch.randn(3, 32, generator=g).to(torch.bfloat16)
    lay = O.w4a16_quantize(w, torch.bfloat16)
    y = O.w8a16_forward(x, lay)
    exact = x.double() @ w.double().t()
    assert y.shape == (3, 12)
    assert float((y.double() - exact).norm() / exact.norm()) < 0.2  # 4-bit weights: coarse but correlated
