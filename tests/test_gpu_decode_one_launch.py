"""The one-launch decode forward (both weight streams in one persistent kernel) against the CPU
oracle and against the two-launch form it replaces."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import build_module

pytestmark = pytest.mark.gpu


def _dev_tensors(case, dev):
    return [v.to(dev) if v is not None else None
            for v in (case.x, case.w_gate, case.b_gate, case.w_up, case.b_up, case.w_down, case.b_down)]


@pytest.mark.parametrize("M", [1, 8, 32, 64])
@pytest.mark.parametrize("K,N,bias", [
    (512, 1024, False),     # fewer phase-2 units than CTAs: some CTAs only contribute to phase 1
    (1024, 3584, True),     # the 8-way tensor-parallel shard width of a 28672 intermediate
    (2048, 7168, False),    # many split tiles in both phases
    (4096, 128, True),      # one phase-1 tile split over 64 CTAs; phase 2 is two reduction blocks per tile
    (256, 18944, False),    # one whole phase-1 tile per CTA on a 148-SM part
])
def test_one_launch_matches_oracle_and_two_launches(pkg, cuda_dev, M, K, N, bias):
    K_ = pkg.ops.kernels
    case = orc.make_case(M, K, N, bias, torch.bfloat16, seed=M + K, w_std=0.5 * K ** -0.5)
    t = _dev_tensors(case, cuda_dev)
    scratch = K_.decode_scratch(M, K, N, torch.bfloat16, cuda_dev)
    y1 = K_.decode_fwd(*t, scratch=scratch, one_launch=True)
    assert pkg._lib.status_read(cuda_dev) == 0
    orc.assert_parity(y1.cpu(), orc.forward_backward(case, grads=False)["y"], "y")
    y2 = K_.decode_fwd(*t, scratch=scratch)
    orc.assert_parity(y1.cpu(), y2.float().cpu(), "one launch vs two", max_abs=2e-2, mean_rel=1e-2)


def test_one_launch_is_repeatable_and_leaves_the_scratch_clean(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    M, K, N = 48, 1024, 4096
    case = orc.make_case(M, K, N, True, torch.bfloat16, seed=3, w_std=0.02)
    t = _dev_tensors(case, cuda_dev)
    scratch = K_.decode_scratch(M, K, N, torch.bfloat16, cuda_dev)
    ys = [K_.decode_fwd(*t, scratch=scratch, one_launch=True) for _ in range(6)]
    assert all(torch.equal(ys[0], y) for y in ys[1:]), "the result must not depend on CTA arrival order"
    # counters of both phases and the two device-wide counts: three 256-byte blocks here
    assert int(scratch[:192].abs().sum()) == 0, "counters must be left at zero"
    # interleaved with the two-launch form on the same scratch
    a = K_.decode_fwd(*t, scratch=scratch)
    b = K_.decode_fwd(*t, scratch=scratch, one_launch=True)
    c = K_.decode_fwd(*t, scratch=scratch)
    assert torch.equal(a, c) and torch.equal(b, ys[0])
    assert pkg._lib.status_read(cuda_dev) == 0


def test_one_launch_with_residual_row_scale_activation_fp16(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    M, K, N = 5, 512, 1536
    case = orc.make_case(M, K, N, True, torch.float16, seed=17, w_std=0.03)
    t = _dev_tensors(case, cuda_dev)
    g = torch.Generator(device="cpu").manual_seed(5)
    res = torch.randn((M, K), generator=g).to(torch.float16).to(cuda_dev)
    rs = (torch.rand((M,), generator=g) + 0.5).to(cuda_dev)
    for act in ("silu", "gelu"):
        y1 = K_.decode_fwd(*t, act=act, residual=res, row_scale=rs, one_launch=True)
        y2 = K_.decode_fwd(*t, act=act, residual=res, row_scale=rs)
        orc.assert_parity(y1.cpu(), y2.float().cpu(), f"{act}: one launch vs two", max_abs=2e-2, mean_rel=1e-2)
    assert pkg._lib.status_read(cuda_dev) == 0


def test_one_launch_replays_from_a_cuda_graph_and_through_the_module(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    case = orc.make_case(8, 512, 1536, True, torch.bfloat16, seed=21, w_std=0.03)
    t = _dev_tensors(case, cuda_dev)
    scratch = K_.decode_scratch(8, 512, 1536, torch.bfloat16, cuda_dev)
    want = K_.decode_fwd(*t, scratch=scratch, one_launch=True)
    torch.cuda.synchronize()
    x_static = t[0].clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_a = K_.decode_fwd(x_static, *t[1:], scratch=scratch, one_launch=True)
        y_b = K_.decode_fwd(y_a, *t[1:], scratch=scratch, one_launch=True)      # chained: dependent launches
    for scale in (1.0, 0.5):
        x_static.copy_(t[0] * scale)
        graph.replay()
        torch.cuda.synchronize()
        ya = K_.decode_fwd(t[0] * scale, *t[1:], scratch=scratch, one_launch=True)
        assert torch.equal(y_a, ya)
        assert torch.equal(y_b, K_.decode_fwd(ya, *t[1:], scratch=scratch, one_launch=True))
    assert torch.equal(K_.decode_fwd(*t, scratch=scratch, one_launch=True), want)

    m = build_module(pkg, case, torch.bfloat16, cuda_dev).eval()
    m.decode_one_launch = True
    with torch.no_grad():
        y = m(case.x.to(cuda_dev))
    assert torch.equal(y, want)
    assert pkg._lib.status_read(cuda_dev) == 0
