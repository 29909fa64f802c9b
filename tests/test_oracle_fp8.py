"""The e4m3 restatement used by the 8-bit decode tests, pinned to values of the format itself
(1 sign, 4 exponent bits with bias 7, 3 mantissa bits; largest finite value 448; no infinities)."""
import torch

from oracle import fp8


def test_e4m3_rounding_known_values():
    x = torch.tensor([0.0, 1.0, 1.0625, 1.1, 1.1875, 240.0, 447.0, 448.0, 500.0, -500.0, 2.0 ** -9, 2.0 ** -10,
                      0.017, 17.0, 18.0, 19.0])
    want = torch.tensor([0.0, 1.0, 1.0, 1.125, 1.25, 240.0, 448.0, 448.0, 448.0, -448.0, 2.0 ** -9, 0.0,
                         0.017578125, 16.0, 18.0, 20.0])
    # 1.0625 and 1.1875 are ties: to even mantissa (1.0 = 1.000b, 1.25 = 1.010b); 2^-9 is the smallest
    # subnormal, 2^-10 a tie between 0 and it (to even: 0); 17 is a tie between 16 and 18 (to 16), 19 -> 20
    assert torch.equal(fp8.e4m3_round(x), want)


def test_row_quantisation_contract():
    g = torch.Generator().manual_seed(0)
    a = torch.randn((5, 256), generator=g) * torch.tensor([0.01, 1.0, 30.0, 1e-6, 0.0])[:, None]
    deq, scale = fp8.quantize_rows(a)
    assert torch.allclose(scale[:4], a.abs().amax(-1)[:4] / 448.0)
    assert scale[4] > 0 and torch.equal(deq[4], torch.zeros(256))
    # the row maximum is represented exactly; every element within half a step of its binade (2^-4 relative)
    assert torch.allclose(deq.abs().amax(-1)[:4], a.abs().amax(-1)[:4], rtol=1e-6)
    big = a[:4].abs() > scale[:4, None] * 2.0 ** -6
    rel = ((deq[:4] - a[:4]).abs() / a[:4].abs().clamp_min(1e-30))[big]
    assert rel.max() <= 2.0 ** -4 + 1e-6


def test_weight_round_trip():
    g = torch.Generator().manual_seed(1)
    w = torch.randn((64, 128), generator=g) * 0.02
    scale = w.abs().amax(1) / 448.0
    w8 = (w / scale[:, None]).to(torch.float8_e4m3fn).view(torch.uint8)
    deq = fp8.dequantize_weight(w8, scale)
    assert (deq - w).abs().max() <= w.abs().amax() * 2.0 ** -4
