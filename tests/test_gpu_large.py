"""Parity at the benchmark configurations' full sizes, where a full CPU oracle run would
take minutes: a sliced oracle instead.

Every row of y and dx depends only on its own token, so a sample of rows is checked
with all of K and N. Every intermediate unit n contributes independently to
dW_gate[n, :], dW_up[n, :], dW_down[:, n], db_gate[n], db_up[n], so a sample of units is
checked over all M rows. db_down is checked in full. Inputs are drawn on the GPU with
the configurations' distributions; the oracle reads the very same 16-bit values back.
"""
import numpy as np
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from oracle import philox

pytestmark = pytest.mark.gpu


def _randn(shape, std, dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(shape, device=dev, generator=g) * std).to(torch.bfloat16)


def _print_report(title, report):
    """The literal and the contract's error figures of every tensor compared (shown with pytest -s or -rP)."""
    print(f"\n{title}")
    for name, r in report:
        print(f"  {name:16s} max abs {r['max_abs']:.3e} (scaled {r['max_abs_scaled']:.3e})  mean rel {r['mean_rel']:.3e}  "
              f"rms(want) {r['rms_want']:.3g}  max|want| {r['max_want']:.3g}")


def _sliced_check(pkg, dev, M, K, N, bias, p, w_std, dy_std, backward, n_rows=128, n_quads=8, seed=0):
    seed_p, offset = 0x5EED, 1
    report = []
    x = _randn((M, K), 1.0, dev, seed)
    m = pkg.FusedGatedMLP(K, N, bias=bias, dropout_p=p).to(dev).to(torch.bfloat16)
    with torch.no_grad():
        for i, prm in enumerate(m.parameters()):
            prm.copy_(_randn(prm.shape, w_std, dev, seed + 1 + i))
    m.train(backward)
    m.set_philox(seed_p, offset)
    if backward:
        dy = _randn((M, K), dy_std, dev, seed + 20)
        xr = x.detach().requires_grad_(True)
        y = m(xr)
        y.backward(dy)
    else:
        with torch.no_grad():
            y = m(x)
    torch.cuda.synchronize()

    f = lambda t: None if t is None else t.detach().float().cpu()
    wg, wu, wd = f(m.gate_proj.weight), f(m.up_proj.weight), f(m.down_proj.weight)
    bg, bu, bd = f(m.gate_proj.bias), f(m.up_proj.bias), f(m.down_proj.bias)
    rng = np.random.default_rng(seed)

    # ---- rows: y (and dx) with all of K and N
    rows = np.sort(rng.choice(M, size=min(n_rows, M), replace=False))
    rows[0], rows[-1] = 0, M - 1
    ridx = torch.from_numpy(rows).to(dev)
    xs = f(x[ridx])
    ks = None
    if backward and p > 0:
        keep = np.stack([philox.keep_mask(1, N, p, seed_p, offset, row0=int(r), n_global=N)[0] for r in rows])
        ks = torch.from_numpy(keep.astype(np.float32) * philox.scale(p))
    orc.assert_parity(f(y[ridx]), orc.forward(xs, wg, bg, wu, bu, wd, bd, ks), "y rows", report=report)
    if not backward:
        _print_report(f"M={M} K={K} N={N} forward", report)
        return
    dys = f(dy[ridx])
    h, g, u = orc.hidden_forward(xs, wg, bg, wu, bu, ks)
    dh = dys @ wd
    if ks is not None:
        dh = dh * ks
    dx_want, _, _, _, _ = orc.hidden_backward(xs, wg, wu, g, u, dh)
    orc.assert_parity(f(xr.grad[ridx]), dx_want, "dx rows", report=report)

    # ---- intermediate units: weight / bias gradients over all M rows
    quads = np.sort(rng.choice(N // 8, size=n_quads, replace=False))   # groups of 8 consecutive units
    cols = (quads[:, None] * 8 + np.arange(8)[None, :]).reshape(-1)
    cidx = torch.from_numpy(cols).to(dev)
    xf, dyf = f(x), f(dy)
    gs = xf @ wg[cols].T + (bg[cols] if bg is not None else 0)
    us = xf @ wu[cols].T + (bu[cols] if bu is not None else 0)
    dhs = dyf @ wd[:, cols]
    hs = orc.silu(gs) * us
    if p > 0:
        keep = np.concatenate([philox.keep_mask(M, 8, p, seed_p, offset, col0=int(q) * 8, n_global=N) for q in quads],
                              axis=1)
        kcs = torch.from_numpy(keep.astype(np.float32) * philox.scale(p))
        dhs, hs = dhs * kcs, hs * kcs
    d_gate = dhs * us * orc.silu_prime(gs)
    d_up = dhs * orc.silu(gs)
    orc.assert_parity(f(m.gate_proj.weight.grad[cidx]), d_gate.T @ xf, "dW_gate units", report=report)
    orc.assert_parity(f(m.up_proj.weight.grad[cidx]), d_up.T @ xf, "dW_up units", report=report)
    orc.assert_parity(f(m.down_proj.weight.grad[:, cidx]), dyf.T @ hs, "dW_down units", report=report)
    if bias:
        orc.assert_parity(f(m.gate_proj.bias.grad[cidx]), d_gate.sum(0), "db_gate units", report=report)
        orc.assert_parity(f(m.up_proj.bias.grad[cidx]), d_up.sum(0), "db_up units", report=report)
        orc.assert_parity(f(m.down_proj.bias.grad), dyf.sum(0), "db_down", report=report)
    _print_report(f"M={M} K={K} N={N} forward+backward", report)


def test_llama8b_forward_full_size(pkg, cuda_dev):
    """M=8192, K=4096, N=14336, no bias, no dropout; x ~ N(0,1), W ~ N(0,0.02)."""
    _sliced_check(pkg, cuda_dev, 8192, 4096, 14336, False, 0.0, 0.02, 0.0, backward=False)


def test_training_shape_all_gradients_full_size(pkg, cuda_dev):
    """M=16384, K=2048, N=8192, bias ~ N(0,0.02), dropout 0.1, dY ~ N(0,1e-2): all seven gradients."""
    _sliced_check(pkg, cuda_dev, 16384, 2048, 8192, True, 0.1, 0.02, 1e-2, backward=True)


def test_large_prefill_forward_backward_full_size(pkg, cuda_dev):
    """M=65536, K=8192, N=28672, W ~ N(0,0.01), dY ~ N(0,1e-2); about 26 GB on the device."""
    _sliced_check(pkg, cuda_dev, 65536, 8192, 28672, False, 0.0, 0.01, 1e-2, backward=True, n_rows=48, n_quads=3)
    torch.cuda.empty_cache()


def test_dropout_mask_at_training_size_is_bit_exact(pkg, cuda_dev):
    K_ = pkg.ops.kernels
    M, N, p, seed, off = 16384, 8192, 0.1, 0x5EED, 0
    got = K_.dropout_mask(M, N, K_.Dropout(p, seed, off), device=cuda_dev)
    for r0, n in ((0, 512), (M - 512, 512)):
        want = philox.keep_mask(n, N, p, seed, off, row0=r0)
        assert np.array_equal(got[r0:r0 + n].cpu().numpy().astype(bool), want)
    assert abs(got.float().mean().item() - 0.9) < 1e-3


def test_decode_config_full_size(pkg, cuda_dev):
    """M in {1, 8, 32, 64}, K=8192, N=28672: the decode path against a full fp32 oracle."""
    K, N = 8192, 28672
    m = pkg.FusedGatedMLP(K, N, bias=False).to(cuda_dev).to(torch.bfloat16).eval()
    with torch.no_grad():
        for i, prm in enumerate(m.parameters()):
            prm.copy_(_randn(prm.shape, 0.02, cuda_dev, 40 + i))
    wg, wu, wd = (t.detach().float().cpu() for t in (m.gate_proj.weight, m.up_proj.weight, m.down_proj.weight))
    for M in (1, 8, 32, 64):
        x = _randn((M, K), 1.0, cuda_dev, M)
        with torch.no_grad():
            y = m(x)
        report = []
        orc.assert_parity(y.cpu(), orc.forward(x.float().cpu(), wg, None, wu, None, wd, None), f"decode M={M}",
                          report=report)
        _print_report(f"decode K={K} N={N}", report)
