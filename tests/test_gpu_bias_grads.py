"""Bias gradients taken inside the weight-gradient GEMMs (row sums of the kernels' own A operand) against
fp32 column sums, over shapes that exercise one and many column tiles, ragged edges, the single-CTA and the
CTA-pair kernel, and repeated calls on one scratch buffer."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import build_module

pytestmark = pytest.mark.gpu

SHAPES = [
    # M (tokens), K (hidden), N (intermediate)
    (64, 64, 128),        # one tile, one reduction block, single-CTA kernel for both GEMMs
    (200, 256, 384),      # ragged token count; dW_gate/up on the pair kernel, one column tile each
    (1000, 768, 1288),    # several column tiles; N and K not multiples of the 256-row tiles
    (4096, 2048, 1024),   # many reduction blocks per column tile
    (130, 520, 72),       # N smaller than one tile half
]


def _close(got, want, dtype):
    tol = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -10
    err = (got.float().cpu() - want).abs().max().item()
    return err <= tol * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("M,K,N", SHAPES)
def test_fused_bias_gradients_match_column_sums(pkg, cuda_dev, M, K, N, dtype):
    K_ = pkg.ops.kernels
    g = torch.Generator(device="cpu").manual_seed(M + K + N)
    d_gate = (torch.randn((M, N), generator=g) * 0.1).to(dtype)
    d_up = (torch.randn((M, N), generator=g) * 0.1).to(dtype)
    dy = (torch.randn((M, K), generator=g) * 0.1).to(dtype)
    x = torch.randn((M, K), generator=g).to(dtype)
    h = torch.randn((M, N), generator=g).to(dtype)
    dev = lambda t: t.to(cuda_dev)
    for rep in range(2):   # the second call finds the scratch as the first one left it
        dwg, dwu, dbg, dbu = K_.bwd_dw_gate_up(dev(d_gate), dev(d_up), dev(x), bias_grads=True)
        dwd, dbd = K_.bwd_dw_down(dev(dy), dev(h), bias_grad=True)
        torch.cuda.synchronize()
        for name, got, want in (("db_gate", dbg, d_gate.float().sum(0)), ("db_up", dbu, d_up.float().sum(0)),
                                ("db_down", dbd, dy.float().sum(0))):
            ok, err = _close(got, want, dtype)
            assert ok, f"{name} (call {rep}): max err {err:.3e}"
        # the GEMM results themselves are those of the plain entry points, bit for bit
        pg, pu = K_.bwd_dw_gate_up(dev(d_gate), dev(d_up), dev(x))
        assert torch.equal(dwg, pg) and torch.equal(dwu, pu)
        assert torch.equal(dwd, K_.bwd_dw_down(dev(dy), dev(h)))
    # stand-alone column sums agree to within the rounding of the 16-bit result
    assert _close(K_.colsum(dev(d_gate)), d_gate.float().sum(0), dtype)[0]


def test_fused_bias_gradients_are_repeatable(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    g = torch.Generator(device=cuda_dev).manual_seed(3)
    d_gate = (torch.randn((8192, 2048), device=cuda_dev, generator=g) * 0.1).to(torch.bfloat16)
    d_up = (torch.randn((8192, 2048), device=cuda_dev, generator=g) * 0.1).to(torch.bfloat16)
    x = torch.randn((8192, 1024), device=cuda_dev, generator=g).to(torch.bfloat16)
    a = K_.bwd_dw_gate_up(d_gate, d_up, x, bias_grads=True)
    b = K_.bwd_dw_gate_up(d_gate, d_up, x, bias_grads=True)
    assert all(torch.equal(p, q) for p, q in zip(a, b))


def test_bias_gradients_stay_right_over_several_steps(pkg, cuda_dev):
    """The two weight-gradient kernels of a module share one scratch buffer. With more than 4096 intermediate
    columns the gate/up kernel's arrival counters reach past the down kernel's, so the down kernel's partial
    sums must not start where its own counters end: every step after the first would find db_up's counters
    dirty. Three steps on one module, all seven gradients against the oracle each time."""
    M, K, N = 256, 256, 8192 + 512
    case = orc.make_case(M, K, N, True, torch.bfloat16, seed=41, w_std=0.5 * K ** -0.5, dy_std=0.05)
    want = orc.forward_backward(case)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev).train()
    for step in range(3):
        m.zero_grad(set_to_none=True)
        x = case.x.to(cuda_dev).requires_grad_(True)
        m(x).backward(case.dy.to(cuda_dev))
        for name, q in m.named_parameters():
            orc.assert_parity(q.grad.cpu(), want["d" + name], f"step {step} d{name}")
    assert pkg._lib.status_read(cuda_dev) == 0

