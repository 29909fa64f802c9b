"""The tcgen05 GEMM engine against torch fp32 matmul, for every operand layout the
forward and backward passes use, including ragged edges (M, N, K not multiples of
the 128 x 256 x 64 tile)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [
    (128, 256, 64),      # one tile, one reduction block
    (128, 256, 512),     # ring wraps (8 blocks through 4 stages)
    (256, 512, 192),     # 2 x 2 tiles
    (200, 328, 136),     # ragged everywhere (multiples of 8)
    (1, 8, 8),           # smallest legal problem
    (1536, 2304, 1024),  # more tiles than fit one wave of TMEM buffers per CTA
    (148 * 128 * 3, 256, 128),  # three tiles per CTA on a 148-SM part: both accumulators reused
]


def _operands(M, N, K, a_mn, b_mn, dtype, dev):
    g = torch.Generator(device="cpu").manual_seed(M * 7 + N * 3 + K)
    a = (torch.randn((M, K), generator=g) * 0.5).to(dtype)
    b = (torch.randn((N, K), generator=g) * 0.5).to(dtype)
    ref = a.float() @ b.float().T
    a_dev = (a.T.contiguous() if a_mn else a).to(dev)
    b_dev = (b.T.contiguous() if b_mn else b).to(dev)
    return a_dev, b_dev, ref


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
@pytest.mark.parametrize("shape", SHAPES)
def test_gemm_layouts(pkg, cuda_dev, shape, a_mn, b_mn, dtype):
    M, N, K = shape
    if a_mn and M % 8:
        pytest.skip("an M-contiguous A needs M % 8 == 0 (16-byte row pitch)")
    if M > 4096 and dtype == torch.float16:
        pytest.skip("large case once")
    a, b, ref = _operands(M, N, K, a_mn, b_mn, dtype, cuda_dev)
    c = pkg.ops.kernels.gemm(a, b, a_mn=a_mn, b_mn=b_mn).float().cpu()
    # fp32 accumulation; the only rounding is the 16-bit store
    tol = 2 ** -8 if dtype == torch.bfloat16 else 2 ** -10
    err = (c - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= tol * max(scale, 1.0), f"max err {err:.3e} at scale {scale:.3e}"


def test_gemm_bias(pkg, cuda_dev):
    a, b, ref = _operands(300, 264, 320, False, False, torch.bfloat16, cuda_dev)
    bias = torch.linspace(-1, 1, 264).to(torch.bfloat16)
    c = pkg.ops.kernels.gemm(a, b, bias=bias.to(cuda_dev)).float().cpu()
    ref = ref + bias.float()
    assert (c - ref).abs().max().item() <= 2 ** -8 * max(ref.abs().max().item(), 1.0)


def test_gemm_is_deterministic(pkg, cuda_dev):
    a, b, _ = _operands(1024, 1024, 512, False, True, torch.bfloat16, cuda_dev)
    c1 = pkg.ops.kernels.gemm(a, b, b_mn=True)
    c2 = pkg.ops.kernels.gemm(a, b, b_mn=True)
    assert torch.equal(c1, c2)


def test_output_slices_and_sm_limit(pkg, cuda_dev):
    """The down projection and dx written chunk by chunk into slices of one buffer, on a reduced
    number of SMs (what the chunked tensor-parallel path does), give the bits of the one-shot call."""
    K_ = pkg.ops.kernels
    g = torch.Generator(device="cpu").manual_seed(5)
    M, K, N = 640, 256, 384
    h = (torch.randn((M, N), generator=g) * 0.5).to(torch.bfloat16).to(cuda_dev)
    wd = (torch.randn((K, N), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    bd = (torch.randn((K,), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    res = (torch.randn((M, K), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    whole = K_.down_fwd(h, wd, bd, res)
    out = torch.empty_like(whole)
    assert pkg._lib.set_sm_limit(100) == 0
    try:
        for r0 in range(0, M, 256):
            r1 = min(M, r0 + 256)
            assert K_.down_fwd(h[r0:r1], wd, bd, res[r0:r1], out=out[r0:r1]).data_ptr() == out[r0:r1].data_ptr()
    finally:
        assert pkg._lib.set_sm_limit(0) == 100
    assert torch.equal(out, whole)

    dg = (torch.randn((M, N), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    du = (torch.randn((M, N), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    wg, wu = ((torch.randn((N, K), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev) for _ in range(2))
    whole = K_.bwd_dx(dg, du, wg, wu)
    out = torch.empty_like(whole)
    for r0 in range(0, M, 256):
        r1 = min(M, r0 + 256)
        K_.bwd_dx(dg[r0:r1], du[r0:r1], wg, wu, out=out[r0:r1])
    assert torch.equal(out, whole)
    with pytest.raises(ValueError):
        K_.bwd_dx(dg, du, wg, wu, out=out[:128])          # wrong shape
    with pytest.raises(ValueError):
        K_.down_fwd(h, wd, bd, out=torch.empty((M, K), dtype=torch.float16, device=cuda_dev))


def test_per_call_tuning_from_two_threads(pkg, cuda_dev):
    """Two host threads launch GEMMs on two streams at once, one with a per-call tuning word (32 SMs, single-CTA
    kernel, raster group 2), the other with the defaults. Both get the bits of an undisturbed call, and the
    process-wide defaults never move: a module that limits its own grids does not change anybody else's."""
    import threading

    K_, L = pkg.ops.kernels, pkg._lib
    lib = L.load()
    g = torch.Generator(device="cpu").manual_seed(9)
    M, K, N = 1024, 512, 768
    h = (torch.randn((M, N), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    wd = (torch.randn((K, N), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    want = K_.down_fwd(h, wd, None)
    torch.cuda.synchronize()
    word = L.tune_word(pair_mode=1, raster_group=2, sm_limit=32)
    before = (lib.gmlp_set_cta_pair_mode(-1), lib.gmlp_set_raster_group(-1), lib.gmlp_set_sm_limit(-1))
    results, errors = {}, []

    def work(name, tuning):
        try:
            with torch.cuda.stream(torch.cuda.Stream(cuda_dev)):
                outs = [K_.down_fwd(h, wd, None, tuning=tuning) for _ in range(20)]
                torch.cuda.current_stream(cuda_dev).synchronize()
            results[name] = outs
        except Exception as e:  # surfaced in the main thread
            errors.append(e)

    threads = [threading.Thread(target=work, args=("tuned", word)), threading.Thread(target=work, args=("plain", 0))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for outs in results.values():
        assert all(torch.equal(o, want) for o in outs)
    assert (lib.gmlp_set_cta_pair_mode(-1), lib.gmlp_set_raster_group(-1), lib.gmlp_set_sm_limit(-1)) == before


def test_wide_and_narrow_tiles_give_the_same_bits(pkg, cuda_dev):
    """Plain-store GEMMs take 256 x 512 tiles per CTA pair when that shortens the schedule (here: the
    down-projection weight gradient of the training shape, 128 wide tiles against 256 narrow ones on 74 pairs).
    Every output element is the same sequence of MMAs either way, so the per-call switch must not change a bit,
    with and without the bias sums taken on the side."""
    K_ = pkg.ops.kernels
    narrow = pkg._lib.tune_word(narrow_tiles=True)
    g = torch.Generator(device="cpu").manual_seed(11)
    M, K, N = 4096, 2048, 8192
    dy = (torch.randn((M, K), generator=g) * 0.05).to(torch.bfloat16).to(cuda_dev)
    h = torch.randn((M, N), generator=g).to(torch.bfloat16).to(cuda_dev)
    assert torch.equal(K_.bwd_dw_down(dy, h), K_.bwd_dw_down(dy, h, tuning=narrow))
    w1, b1 = K_.bwd_dw_down(dy, h, bias_grad=True)
    w2, b2 = K_.bwd_dw_down(dy, h, bias_grad=True, tuning=narrow)
    assert torch.equal(w1, w2) and torch.equal(b1, b2)
    ref = dy.float().t() @ h.float()
    assert (w1.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.abs().max().item())
    # ragged: the second half of the last wide tile lies outside the matrix
    h2 = h[:, :8192 - 256 - 64].contiguous()
    assert torch.equal(K_.bwd_dw_down(dy, h2), K_.bwd_dw_down(dy, h2, tuning=narrow))
    assert pkg._lib.status_read(cuda_dev) == 0

