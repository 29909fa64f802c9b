"""fp32 modules (tf32 products): the recipes of the reference's own tests, unchanged in dtype
(tests/test_gated_mlp_fwd.py:23-38, tests/test_gated_mlp_bwd.py:27-80 and :89-129: default-constructed
modules in float32, torch.rand inputs), held to the tolerance class those tests use on a GPU (atol 1e-3),
against the fp32 CPU oracle. The tensor core takes the top 19 bits of each fp32 operand (tf32: 10 mantissa
bits, truncated), so a product is short by up to 2^-10 relative per operand and sums of like-signed terms
come out a few parts in 10^3 small: the bounds below are relative to the size of the values."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import build_module

pytestmark = pytest.mark.gpu


def _rel(got, want):
    return ((got.float().cpu() - want).norm() / want.norm()).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 136), (1024, 768, 512), (8, 8, 8)])
def test_tf32_gemm_against_fp32_matmul(pkg, cuda_dev, M, N, K):
    g = torch.Generator().manual_seed(M + N + K)
    a, b = torch.randn((M, K), generator=g), torch.randn((N, K), generator=g)
    bias = torch.randn((N,), generator=g)
    c = pkg.ops.kernels.gemm(a.to(cuda_dev), b.to(cuda_dev), bias=bias.to(cuda_dev))
    assert c.dtype == torch.float32
    want = a @ b.T + bias
    scale = (a.abs() @ b.abs().T).max().item()      # sum of |terms|: what the operand truncation scales with
    assert (c.cpu() - want).abs().max().item() <= 2.0 ** -9 * scale
    # operands given transposed are handled by the wrapper
    c2 = pkg.ops.kernels.gemm(a.t().contiguous().to(cuda_dev), b.t().contiguous().to(cuda_dev), a_mn=True, b_mn=True)
    assert (c2.cpu() - a @ b.T).abs().max().item() <= 2.0 ** -9 * scale


def test_reference_forward_test_recipe(pkg, cuda_dev):
    """test_gated_mlp_fwd: default module (K=256, N=512, bias), float32, x = rand(128, K)."""
    torch.manual_seed(0)
    m = pkg.FusedGatedMLP(dropout_p=0.0).to(cuda_dev).to(torch.float32)
    x = torch.rand((128, m.hidden_size))
    y = m(x.to(cuda_dev))
    assert y.dtype == torch.float32
    sd = {k: v.detach().cpu() for k, v in m.state_dict().items()}
    want = orc.forward(x, sd["gate_proj.weight"], sd["gate_proj.bias"], sd["up_proj.weight"], sd["up_proj.bias"],
                       sd["down_proj.weight"], sd["down_proj.bias"])
    torch.testing.assert_close(y.detach().cpu(), want, atol=1e-3, rtol=1e-3)


def test_reference_backward_test_recipe(pkg, cuda_dev):
    """test_gated_mlp_bwd: bias=False, float32, x = rand(16, 32, K); autograd.grad w.r.t. (x, up.weight, gate.weight)."""
    torch.manual_seed(1)
    m = pkg.FusedGatedMLP(dropout_p=0.0, bias=False).to(cuda_dev).to(torch.float32)
    x = torch.rand((16, 32, m.hidden_size))
    go = torch.rand_like(x)
    xd = x.to(cuda_dev).requires_grad_(True)
    out = m(xd)
    gx, gu, gg = torch.autograd.grad(out, (xd, m.up_proj.weight, m.gate_proj.weight), grad_outputs=go.to(cuda_dev),
                                     retain_graph=True, allow_unused=True)
    sd = {k: v.detach().cpu() for k, v in m.state_dict().items()}
    want_y = orc.forward(x, sd["gate_proj.weight"], None, sd["up_proj.weight"], None, sd["down_proj.weight"], None)
    torch.testing.assert_close(out.detach().cpu(), want_y, atol=1e-3, rtol=1e-3)
    want = orc.backward(x, sd["gate_proj.weight"], None, sd["up_proj.weight"], None, sd["down_proj.weight"], None, go)
    assert _rel(gx, want["dx"]) < 4e-3          # all-positive inputs: the truncation errors add up in one direction
    assert _rel(gu, want["dup_proj.weight"]) < 4e-3
    assert _rel(gg, want["dgate_proj.weight"]) < 4e-3
    # a second walk over the same graph is allowed on this path (nothing is overwritten)
    torch.autograd.grad(out, (xd,), grad_outputs=go.to(cuda_dev))


def test_reference_op_level_recipe(pkg, cuda_dev):
    """test_bwd_ops_triton: B, M, N, K = 2, 32, 512, 256; every operand rand / K; float32."""
    B, M, N, K = 2, 32, 512, 256
    g = torch.Generator().manual_seed(2)
    x = torch.rand((B * M, K), generator=g) / K
    W_up = torch.rand((N, K), generator=g) / K
    W_gp = torch.rand((N, K), generator=g) / K
    grad_output = torch.rand((B * M, N), generator=g) / K
    h, gq, uq = orc.hidden_forward(x, W_gp, None, W_up, None)
    dx_ref, dW_up_ref, dW_gp_ref, _, _ = orc.hidden_backward(x, W_gp, W_up, gq, uq, grad_output)
    dev = lambda t: t.to(cuda_dev)
    hh = pkg.mlp_hidden_states_fwd(dev(x), dev(W_up), None, dev(W_gp), None, "silu", 0.0)
    assert _rel(hh, h) < 4e-3
    dx, dW_up, dW_gp = pkg.mlp_hidden_states_bwd(dev(x), dev(W_up), dev(W_gp), dev(grad_output))
    assert _rel(dx, dx_ref) < 4e-3 and _rel(dW_up, dW_up_ref) < 4e-3 and _rel(dW_gp, dW_gp_ref) < 4e-3


def test_all_seven_gradients_with_bias_and_dropout_in_fp32(pkg, cuda_dev):
    M, K, N, p = 520, 384, 640, 0.1
    case = orc.make_case(M, K, N, True, torch.float32, seed=9, w_std=0.5 * K ** -0.5, dy_std=0.05)
    m = build_module(pkg, case, torch.float32, cuda_dev, dropout_p=p).train()
    m.set_philox(0x5EED, 4)
    x = case.x.to(cuda_dev).requires_grad_(True)
    y = m(x)
    y.backward(case.dy.to(cuda_dev))
    want = orc.forward_backward(case, dropout_p=p, seed=0x5EED, offset=4)
    got = {"y": y, "dx": x.grad, **{"d" + n: q.grad for n, q in m.named_parameters()}}
    assert set(got) == set(want)
    for k, v in want.items():
        assert _rel(got[k].detach(), v) < 4e-3, k
