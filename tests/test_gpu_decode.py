"""Skinny-M (decode) forward: the weight-streaming kernels against the CPU oracle,
including shapes whose row tiles are split across CTAs in every possible way."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import build_module

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M", [1, 8, 32, 64])
@pytest.mark.parametrize("K,N,bias", [
    (512, 1024, False),     # fewer work units than SMs in the down projection
    (1024, 3584, True),     # the 8-way tensor-parallel shard width of a 28672 intermediate
    (2048, 7168, False),    # many split tiles in both kernels
    (4096, 128, True),      # one gate/up tile split over 64 CTAs: the fix-up sums 64 partial tiles
    (256, 18944, False),    # 148 gate/up row tiles: one whole tile per CTA on a 148-SM part, nothing split
    (256, 24576, True),     # 192 row tiles: every CTA owns a whole tile, the other 44 are split over all CTAs
])
def test_decode_matches_oracle(pkg, cuda_dev, M, K, N, bias):
    case = orc.make_case(M, K, N, bias, torch.bfloat16, seed=M + K, w_std=0.5 * K ** -0.5)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev).eval()
    with torch.no_grad():
        y = m(case.x.to(cuda_dev))
    assert m._decode_scratch is not None, "the decode path was not taken"
    orc.assert_parity(y.cpu(), orc.forward_backward(case, grads=False)["y"], "y")


def test_decode_equals_gemm_path_and_is_repeatable(pkg, cuda_dev):
    """Same inputs through the tile-GEMM kernels (M padded into a 128-row tile) and the
    streaming kernels; the streaming result must not depend on CTA arrival order."""
    K_ = pkg.ops.kernels
    case = orc.make_case(48, 1024, 4096, True, torch.bfloat16, seed=3, w_std=0.02)
    t = [v.to(cuda_dev) if v is not None else None
         for v in (case.x, case.w_gate, case.b_gate, case.w_up, case.b_up, case.w_down, case.b_down)]
    y_gemm = K_.down_fwd(K_.hidden_fwd(t[0], t[1], t[2], t[3], t[4]), t[5], t[6])
    scratch = K_.decode_scratch(48, 1024, 4096, torch.bfloat16, cuda_dev)
    ys = [K_.decode_fwd(*t, scratch=scratch) for _ in range(5)]
    assert all(torch.equal(ys[0], y) for y in ys[1:])
    # counter area: one int per 128-row weight tile of each kernel, each block padded to 256 bytes
    n_counters = (256 + 256) // 4
    assert int(scratch[:n_counters].abs().sum()) == 0, "counters must be left at zero"
    orc.assert_parity(ys[0].cpu(), y_gemm.float().cpu(), "decode vs gemm", max_abs=2e-2, mean_rel=1e-2)


@pytest.mark.parametrize("act", ["gelu", "relu", "no_act"])
def test_decode_other_activations(pkg, cuda_dev, act):
    case = orc.make_case(16, 256, 1024, True, torch.bfloat16, seed=31, w_std=0.03)
    K, N = 256, 1024
    m = pkg.FusedGatedMLP(K, N, bias=True, hidden_act=act)
    m.load_state_dict(case.state_dict())
    m = m.to(cuda_dev).to(torch.bfloat16).eval()
    with torch.no_grad():
        y = m(case.x.to(cuda_dev))
    assert m._decode_scratch is not None
    orc.assert_parity(y.cpu(), orc.forward_backward(case, grads=False, act=act)["y"], "y")


def test_decode_fp16_and_3d_input(pkg, cuda_dev):
    case = orc.make_case(0, 256, 512, True, torch.float16, seed=9, lead_shape=(2, 5), w_std=0.03)
    m = build_module(pkg, case, torch.float16, cuda_dev).eval()
    with torch.no_grad():
        y = m(case.x.to(cuda_dev))
    assert y.shape == (2, 5, 256)
    orc.assert_parity(y.cpu(), orc.forward_backward(case, grads=False)["y"], "y")


def test_decode_rejects_what_it_cannot_do(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    z = lambda *s: torch.zeros(s, dtype=torch.bfloat16, device=cuda_dev)
    with pytest.raises(ValueError):
        K_.decode_fwd(z(65, 128), z(256, 128), None, z(256, 128), None, z(128, 256), None)
    with pytest.raises(pkg._lib.GmlpError, match="scratch"):
        K_.decode_fwd(z(4, 128), z(256, 128), None, z(256, 128), None, z(128, 256), None,
                      scratch=torch.zeros(64, dtype=torch.int32, device=cuda_dev))


def test_decode_replays_from_a_cuda_graph(pkg, cuda_dev):
    """The decode path makes no allocation or synchronisation inside the C calls, so a caller can
    capture it once and replay it (what a serving loop with a few tokens per step wants)."""
    K_ = pkg.ops.kernels
    case = orc.make_case(8, 512, 1536, True, torch.bfloat16, seed=21, w_std=0.03)
    t = [v.to(cuda_dev) if v is not None else None
         for v in (case.x, case.w_gate, case.b_gate, case.w_up, case.b_up, case.w_down, case.b_down)]
    scratch = K_.decode_scratch(8, 512, 1536, torch.bfloat16, cuda_dev)
    want = K_.decode_fwd(*t, scratch=scratch)          # also warms up (function attributes, module load)
    torch.cuda.synchronize()
    x_static = t[0].clone()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = K_.decode_fwd(x_static, *t[1:], scratch=scratch)
    for scale in (1.0, 0.5):
        x_static.copy_(t[0] * scale)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y_static, K_.decode_fwd(t[0] * scale, *t[1:], scratch=scratch))
    assert torch.equal(K_.decode_fwd(*t, scratch=scratch), want)


def test_decode_writes_into_given_buffer(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    g = torch.Generator(device="cpu").manual_seed(9)
    M, K, N = 8, 256, 512
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(cuda_dev)
    wg, wu = ((torch.randn((N, K), generator=g) * 0.05).to(torch.bfloat16).to(cuda_dev) for _ in range(2))
    wd = (torch.randn((K, N), generator=g) * 0.05).to(torch.bfloat16).to(cuda_dev)
    want = K_.decode_fwd(x, wg, None, wu, None, wd, None)
    buf = torch.zeros((2 * M, K), dtype=torch.bfloat16, device=cuda_dev)
    got = K_.decode_fwd(x, wg, None, wu, None, wd, None, out=buf[M:])
    assert got.data_ptr() == buf[M:].data_ptr() and torch.equal(got, want)
    assert buf[:M].abs().max().item() == 0


def test_decode_right_after_the_weights_were_written(pkg, cuda_dev):
    """The decode kernels start streaming weights while the kernel ahead of them is still running, unless the
    call asks for an ordinary launch. With that flag a call placed directly behind the kernels that write the
    weights must see the new weights, every time; the module sets the flag by itself when a parameter's
    version counter has moved since its last decode call."""
    K_ = pkg.ops.kernels
    g = torch.Generator(device="cpu").manual_seed(21)
    M, K, N = 16, 2048, 8192
    x = torch.randn((M, K), generator=g).to(torch.bfloat16).to(cuda_dev)
    sets = []
    for _ in range(2):
        wg, wu = ((torch.randn((N, K), generator=g) * 0.03).to(torch.bfloat16).to(cuda_dev) for _ in range(2))
        wd = (torch.randn((K, N), generator=g) * 0.03).to(torch.bfloat16).to(cuda_dev)
        sets.append((wg, wu, wd))
    scratch = K_.decode_scratch(M, K, N, torch.bfloat16, cuda_dev)
    want = [K_.decode_fwd(x, s[0], None, s[1], None, s[2], None, scratch=scratch) for s in sets]
    assert not torch.equal(want[0], want[1])
    live = [t.clone() for t in sets[0]]
    for i in range(1, 13):
        for dst, src in zip(live, sets[i % 2]):
            dst.copy_(src)                                   # the writers: three copy kernels, back to back
        y = K_.decode_fwd(x, live[0], None, live[1], None, live[2], None, scratch=scratch, ordinary_launch=True)
        assert torch.equal(y, want[i % 2]), f"call {i} read weights from before the copy"

    case = orc.make_case(M, 512, 1024, False, torch.bfloat16, seed=5, w_std=0.03)
    m = build_module(pkg, case, torch.bfloat16, cuda_dev).eval()
    seen = []
    real = K_.decode_fwd
    try:
        K_.decode_fwd = lambda *a, **kw: (seen.append(kw.get("ordinary_launch")), real(*a, **kw))[1]
        with torch.no_grad():
            xd = case.x.to(cuda_dev)
            m(xd); m(xd)
            m.up_proj.weight.mul_(1.5)                       # what an optimiser step or a weight merge does
            y = m(xd); m(xd)
    finally:
        K_.decode_fwd = real
    assert seen == [True, False, True, False]
    import dataclasses
    case2 = dataclasses.replace(case, w_up=(case.w_up.to(torch.bfloat16) * 1.5).to(case.w_up.dtype))
    orc.assert_parity(y.cpu(), orc.forward_backward(case2, grads=False)["y"], "y after the update")
