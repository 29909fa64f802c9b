"""RMSNorm in front of the MLP (module.attach_input_norm): the inference path (1 / rms applied to the
gate/up kernel's accumulators, norm weight folded into the weights; tile kernels and decode kernels) and the
training path (normalised activations materialised, row-wise backward kernel) against the CPU oracle, which
is pinned to torch.nn.RMSNorm + the reference's eager module by the fixture norm_mlp_bf16."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import build_module, load_golden

pytestmark = pytest.mark.gpu


def _norm_weight(K, seed):
    g = torch.Generator().manual_seed(seed)
    return (1.0 + 0.2 * torch.randn(K, generator=g)).to(torch.bfloat16)


def test_row_statistics_and_backward_kernels(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    g = torch.Generator().manual_seed(1)
    for M, K in ((1, 64), (37, 264), (520, 4096)):
        x = (torch.randn((M, K), generator=g) * 2.0).to(torch.bfloat16)
        rs, xn = K_.rms_rowscale(x.to(cuda_dev), 1e-5, normalised=True)
        want_rs = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        torch.testing.assert_close(rs.cpu(), want_rs, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(xn.float().cpu(), x.float() * want_rs[:, None], rtol=2 ** -8, atol=1e-6)
        assert torch.equal(K_.rms_rowscale(x.to(cuda_dev), 1e-5), rs)
        dxn = (torch.randn((M, K), generator=g) * 0.1).to(torch.bfloat16)
        dx = K_.rms_bwd(dxn.to(cuda_dev), xn, rs)
        xnf, df = xn.float().cpu(), dxn.float()
        want = want_rs[:, None] * (df - xnf * (df * xnf).mean(-1, keepdim=True))
        orc.assert_parity(dx.cpu(), want, f"rms_bwd {M}x{K}")


@pytest.mark.parametrize("M", [8, 64, 300])   # 8 and 64 tokens take the decode kernels, 300 the tile GEMMs
def test_norm_prologue_inference(pkg, cuda_dev, M):
    K, N = 256, 512
    case = orc.make_case(M, K, N, True, torch.bfloat16, seed=M, w_std=0.5 * K ** -0.5)
    w = _norm_weight(K, 3)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev).eval()
    m.attach_input_norm(w, eps=1e-5)
    x = (case.x.float() * 3.0).to(torch.bfloat16)      # rms well away from 1
    with torch.no_grad():
        y = m(x.to(cuda_dev))
    assert (m._decode_scratch is not None) == (M <= 64)
    # the engine folds the norm weight into 16-bit copies of W_gate / W_up: the oracle gets those copies
    f = lambda t: None if t is None else t.float()
    wg = (case.w_gate.to(cuda_dev) * w.to(cuda_dev)).cpu().float()
    wu = (case.w_up.to(cuda_dev) * w.to(cuda_dev)).cpu().float()
    xs = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5)
    want = orc.forward(xs, wg, f(case.b_gate), wu, f(case.b_up), f(case.w_down), f(case.b_down))
    orc.assert_parity(y.cpu(), want, f"norm + MLP, M={M}")
    # and within the (looser) distance the 16-bit folding itself allows, the unfolded definition
    full = orc.forward(orc.rmsnorm(x.float(), w.float(), 1e-5), f(case.w_gate), f(case.b_gate), f(case.w_up),
                       f(case.b_up), f(case.w_down), f(case.b_down))
    orc.assert_parity(y.cpu(), full, f"norm + MLP vs unfolded, M={M}", max_abs=4e-2, mean_rel=2e-2)
    # a changed parameter refreshes the folded copies
    with torch.no_grad():
        m.input_norm_weight.mul_(2.0)
        y2 = m(x.to(cuda_dev))
    assert not torch.equal(y, y2)


def test_norm_training_matches_fixture(pkg, cuda_dev):
    t, meta, dt = load_golden("norm_mlp_bf16")
    K, N = t["p.gate_proj.weight"].shape[1], t["p.gate_proj.weight"].shape[0]
    m = pkg.FusedGatedMLP(K, N, bias=True)
    m.load_state_dict({k[2:]: v.float() for k, v in t.items() if k.startswith("p.")})
    m = m.to(cuda_dev).to(dt)
    m.attach_input_norm(t["norm_weight"], eps=float(meta["eps"]))
    x = t["x"].to(cuda_dev).requires_grad_(True)
    y = m(x)
    y.backward(t["dy"].to(cuda_dev))
    orc.assert_parity(y.cpu(), t["y"], "y")
    orc.assert_parity(x.grad.cpu(), t["dx"], "dx")
    for name, p in m.named_parameters():
        orc.assert_parity(p.grad.cpu(), t["d" + name], "d" + name)


def test_norm_training_larger_shape(pkg, cuda_dev):
    M, K, N = 1024, 512, 1536
    case = orc.make_case(M, K, N, True, torch.bfloat16, seed=77, w_std=0.5 * K ** -0.5, dy_std=0.05)
    w = _norm_weight(K, 5)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev)
    m.attach_input_norm(w, eps=1e-6)
    x = case.x.to(cuda_dev).requires_grad_(True)
    y = m(x)
    y.backward(case.dy.to(cuda_dev))
    want = orc.norm_forward_backward(case, w, 1e-6)
    orc.assert_parity(y.cpu(), want["y"], "y")
    orc.assert_parity(x.grad.cpu(), want["dx"], "dx")
    for name, p in m.named_parameters():
        orc.assert_parity(p.grad.cpu(), want["d" + name], "d" + name)
