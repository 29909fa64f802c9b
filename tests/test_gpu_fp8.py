"""Decode with e4m3 weights: the row quantiser bit for bit against its CPU restatement, the two-kernel
forward against the oracle under the same quantisation contract (tight tolerance: what differs is the
order of fp32 additions), and what the activation quantisation itself costs against the same weights
with unquantised activations (stated, loose)."""
import pytest
import torch

from oracle import fp8
from oracle import gated_mlp_oracle as orc

pytestmark = pytest.mark.gpu


def test_row_quantiser_is_bit_exact(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    g = torch.Generator().manual_seed(2)
    x = (torch.randn((37, 1024), generator=g) * torch.logspace(-3, 2, 37)[:, None]).to(torch.bfloat16)
    x[5] = 0
    q, scale = K_.quantize_rows_e4m3(x.to(cuda_dev))
    want_scale = x.float().abs().amax(-1).clamp_min(1e-30) / 448.0
    assert torch.equal(scale.cpu(), want_scale)
    want_q = (x.float() / want_scale[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert torch.equal(q.cpu(), want_q)


def _case(M, K, N, bias, seed):
    case = orc.make_case(M, K, N, bias, torch.bfloat16, seed=seed, w_std=0.5 * K ** -0.5)
    return case


@pytest.mark.parametrize("M,K,N,bias", [(1, 512, 768, False), (8, 512, 768, True), (33, 1024, 512, True),
                                        (64, 256, 1280, False)])
def test_fp8_decode_matches_quantised_oracle(pkg, cuda_dev, M, K, N, bias):
    K_ = pkg.ops.kernels
    case = _case(M, K, N, bias, seed=M + N)
    dev = lambda t: None if t is None else t.to(cuda_dev)
    q = {n: K_.quantize_weight_rows_e4m3(dev(w)) for n, w in (("g", case.w_gate), ("u", case.w_up), ("d", case.w_down))}
    y = K_.decode_fwd_fp8(dev(case.x), q["g"][0], q["g"][1], dev(case.b_gate), q["u"][0], q["u"][1], dev(case.b_up),
                          q["d"][0], q["d"][1], dev(case.b_down))
    deq = {n: fp8.dequantize_weight(w8.cpu(), s.cpu()) for n, (w8, s) in q.items()}
    f = lambda t: None if t is None else t.float()
    want = fp8.decode_forward(case.x.float(), deq["g"], f(case.b_gate), deq["u"], f(case.b_up), deq["d"],
                              f(case.b_down))
    orc.assert_parity(y.cpu(), want, f"fp8 decode M={M}")
    # the price of quantising the activations (same weights, 16-bit activations): a few percent
    ref = fp8.decode_forward(case.x.float(), deq["g"], f(case.b_gate), deq["u"], f(case.b_up), deq["d"],
                             f(case.b_down), quantize_activations=False)
    orc.assert_parity(y.cpu(), ref, f"fp8 decode vs 16-bit activations M={M}", max_abs=3e-1, mean_rel=6e-2)


def test_fp8_decode_full_size_through_the_module(pkg, cuda_dev):
    """K=8192, N=28672 (the decode configuration), M=8, through FusedGatedMLP.quantize_decode_weights()."""
    K, N, M = 8192, 28672, 8
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    m = pkg.FusedGatedMLP(K, N, bias=False).to(cuda_dev).to(torch.bfloat16).eval()
    with torch.no_grad():
        for prm in m.parameters():
            prm.copy_((torch.randn(prm.shape, device=cuda_dev, generator=g) * 0.02).to(torch.bfloat16))
    x = torch.randn((M, K), device=cuda_dev, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        y16 = m(x)
        m.quantize_decode_weights()
        y8 = m(x)
        (wg8, wgs), (wu8, wus), (wd8, wds) = m._fp8
    deq = [fp8.dequantize_weight(a.cpu(), b.cpu()) for a, b in ((wg8, wgs), (wu8, wus), (wd8, wds))]
    want = fp8.decode_forward(x.float().cpu(), deq[0], None, deq[1], None, deq[2], None)
    orc.assert_parity(y8.cpu(), want, "fp8 decode, full size")
    # against the 16-bit path of the same module: weight and activation quantisation together
    orc.assert_parity(y8.cpu(), y16.float().cpu(), "fp8 vs 16-bit decode", max_abs=5e-1, mean_rel=8e-2)
    m.quantize_decode_weights(False)
    with torch.no_grad():
        assert torch.equal(m(x), y16)
