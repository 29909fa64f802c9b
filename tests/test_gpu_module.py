"""Forward/backward parity of FusedGatedMLP against the CPU oracle on seeded inputs,
plus the module-API behaviours the reference's tests rely on."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import build_module

pytestmark = pytest.mark.gpu


def _run(pkg, dev, case, dtype, p=0.0, seed=0, offset=0, train=True):
    m = build_module(pkg, case, dtype, dev, dropout_p=p)
    m.train(train)
    m.set_philox(seed, offset)
    x = case.x.to(dev).requires_grad_(True)
    y = m(x)
    y.backward(case.dy.to(dev))
    got = {"y": y, "dx": x.grad}
    got.update({"d" + n: q.grad for n, q in m.named_parameters()})
    return {k: v.cpu() for k, v in got.items()}, m


CASES = [
    # M, K, N, bias, dtype, p
    (128, 512, 256, False, torch.float16, 0.0),
    (128, 256, 512, True, torch.bfloat16, 0.0),
    (520, 384, 640, True, torch.bfloat16, 0.1),      # ragged M, bias, dropout
    (64, 128, 1024, False, torch.bfloat16, 0.5),
    (1, 256, 256, True, torch.bfloat16, 0.0),        # a single token
    (2048, 1024, 2048, True, torch.bfloat16, 0.1),   # several tiles per CTA
]


@pytest.mark.parametrize("M,K,N,bias,dtype,p", CASES)
def test_forward_backward_parity(pkg, cuda_dev, M, K, N, bias, dtype, p):
    # weights ~ N(0, 1/(4K)) keep activations and outputs O(1), where the absolute tolerance is meaningful
    case = orc.make_case(M, K, N, bias, dtype, seed=M + N, w_std=0.5 * K ** -0.5, dy_std=0.05)
    got, _ = _run(pkg, cuda_dev, case, dtype, p=p, seed=0x5EED, offset=2)
    want = orc.forward_backward(case, dropout_p=p, seed=0x5EED, offset=2)
    assert set(got) == set(want)
    for k in want:
        orc.assert_parity(got[k], want[k], k)


def test_eval_mode_disables_dropout(pkg, cuda_dev):
    case = orc.make_case(96, 128, 256, True, torch.bfloat16, seed=1)
    got, _ = _run(pkg, cuda_dev, case, torch.bfloat16, p=0.3, train=False)
    want = orc.forward_backward(case, dropout_p=0.0)
    orc.assert_parity(got["y"], want["y"], "y")


def test_three_dimensional_input_and_no_grad(pkg, cuda_dev):
    case = orc.make_case(0, 256, 512, True, torch.bfloat16, seed=2, lead_shape=(16, 32))
    m = build_module(pkg, case, torch.bfloat16, cuda_dev)
    with torch.no_grad():
        y = m(case.x.to(cuda_dev))
    assert y.shape == (16, 32, 256)
    orc.assert_parity(y.cpu(), orc.forward_backward(case, grads=False)["y"], "y")


def test_autograd_grad_subset_like_reference_test(pkg, cuda_dev):
    """tests/test_gated_mlp_bwd.py:53-75 of the reference: autograd.grad w.r.t. (x, up.weight, gate.weight)."""
    case = orc.make_case(0, 256, 512, False, torch.bfloat16, seed=4, lead_shape=(16, 32), x_dist="uniform")
    m = build_module(pkg, case, torch.bfloat16, cuda_dev)
    x = case.x.to(cuda_dev).requires_grad_(True)
    out = m(x)
    gx, gu, gg = torch.autograd.grad(out, (x, m.up_proj.weight, m.gate_proj.weight),
                                     grad_outputs=case.dy.to(cuda_dev))
    want = orc.forward_backward(case)
    orc.assert_parity(gx.cpu(), want["dx"], "dx")
    orc.assert_parity(gu.cpu(), want["dup_proj.weight"], "dW_up")
    orc.assert_parity(gg.cpu(), want["dgate_proj.weight"], "dW_gate")
    assert m.down_proj.weight.grad is None


def test_philox_offset_advances_and_is_reproducible(pkg, cuda_dev):
    case = orc.make_case(64, 128, 256, False, torch.bfloat16, seed=5)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev, dropout_p=0.5).train()
    x = case.x.to(cuda_dev)
    m.set_philox(11, 0)
    with torch.no_grad():
        y0, y1 = m(x), m(x)
    assert m.philox_offset == 2 and not torch.equal(y0, y1)
    m.set_philox(11, 0)
    with torch.no_grad():
        assert torch.equal(m(x), y0)


def test_results_are_bitwise_repeatable(pkg, cuda_dev):
    case = orc.make_case(640, 256, 768, True, torch.bfloat16, seed=6)
    a, _ = _run(pkg, cuda_dev, case, torch.bfloat16, p=0.1, seed=1)
    b, _ = _run(pkg, cuda_dev, case, torch.bfloat16, p=0.1, seed=1)
    assert all(torch.equal(a[k], b[k]) for k in a)


def test_host_pipeline_streams_distinct_batches(pkg, cuda_dev):
    """Pinned host batches through HostPipeline (copies and compute on three streams) give the
    same bits as calling the module on each batch directly."""
    case = orc.make_case(256, 256, 512, True, torch.bfloat16, seed=8, w_std=0.03)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev).eval()

    def step(x_dev):
        with torch.no_grad():
            return m(x_dev)

    g = torch.Generator().manual_seed(0)
    xs = [torch.randn((256, 256), generator=g).to(torch.bfloat16).pin_memory() for _ in range(7)]
    ys = [torch.empty((256, 256), dtype=torch.bfloat16).pin_memory() for _ in range(7)]
    pipe = pkg.host_pipeline.HostPipeline(step, cuda_dev, depth=3)
    for x, y in zip(xs, ys):
        pipe.submit(y, x)
    pipe.drain()
    for x, y in zip(xs, ys):
        assert torch.equal(y, step(x.to(cuda_dev)).cpu())
    with pytest.raises(ValueError):
        pipe.submit(torch.empty(4, 4), torch.empty(4, 4))


@pytest.mark.parametrize("M", [8, 300])   # 8 tokens without grad takes the decode kernels, 300 the tile GEMMs
def test_fused_residual(pkg, cuda_dev, M):
    case = orc.make_case(M, 256, 512, True, torch.bfloat16, seed=M, w_std=0.03, dy_std=0.05)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev).eval()
    res = (torch.randn((M, 256), generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16)
    want = orc.forward_backward(case)
    with torch.no_grad():
        y = m(case.x.to(cuda_dev), residual=res.to(cuda_dev))
    orc.assert_parity(y.cpu(), want["y"] + res.float(), "y + residual (no grad)")
    x = case.x.to(cuda_dev).requires_grad_(True)
    r = res.to(cuda_dev).requires_grad_(True)
    y = m(x, residual=r)
    y.backward(case.dy.to(cuda_dev))
    orc.assert_parity(y.cpu(), want["y"] + res.float(), "y + residual")
    orc.assert_parity(x.grad.cpu(), want["dx"], "dx")
    assert torch.equal(r.grad, case.dy.to(cuda_dev))
    with pytest.raises(ValueError):
        m(x, residual=r[:, :128])


def test_inplace_backward_reuses_saved_buffers_and_guards_a_second_pass(pkg, cuda_dev):
    """By default d_gate / d_up are written over the saved gate / up pre-activations: same gradients as the
    out-of-place form, less peak memory, and a second backward over the same forward (which would read
    overwritten activations) raises instead of returning wrong numbers. With inplace_backward=False the
    graph can be walked twice."""
    case = orc.make_case(512, 256, 1024, True, torch.bfloat16, seed=21, w_std=0.03, dy_std=0.05)
    dy = case.dy.to(cuda_dev)

    def grads(inplace, twice=False):
        m = build_module(pkg, case, torch.bfloat16, cuda_dev)
        m.inplace_backward = inplace
        x = case.x.to(cuda_dev).requires_grad_(True)
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats(cuda_dev)
        base = torch.cuda.memory_allocated(cuda_dev)
        y = m(x)
        y.backward(dy, retain_graph=twice)
        peak = torch.cuda.max_memory_allocated(cuda_dev) - base
        out = {"dx": x.grad.clone(), **{n: q.grad.clone() for n, q in m.named_parameters()}}
        if twice:
            y.backward(dy)
        return out, peak

    a, peak_in = grads(True)
    b, peak_out = grads(False)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert peak_out - peak_in >= 2 * 512 * 1024 * 2 * 0.9      # two [M, N] 16-bit buffers fewer
    grads(False, twice=True)                                     # allowed
    with pytest.raises(RuntimeError, match="inplace_backward"):
        grads(True, twice=True)
