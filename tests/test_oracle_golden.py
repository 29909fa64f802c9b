"""Pins the CPU oracle against outputs of the reference's own eager implementation
(fixtures made by tests/golden/make_golden.py from the reference checkout)."""
import pytest
import torch

from oracle import gated_mlp_oracle as orc
from _util import golden_params, load_golden

ACTS = ["gelu", "relu", "sigmoid", "tanh", "leaky_relu", "no_act"]
MODULE_FIXTURES = ["c1_readme_fp16", "default_bias_3d_bf16", "dropout_bias_bf16"] + [f"act_{a}_bf16" for a in ACTS]


@pytest.mark.parametrize("name", MODULE_FIXTURES)
def test_oracle_matches_reference_module(name):
    t, meta, _ = load_golden(name)
    f = lambda v: None if v is None else v.float()
    wg, bg, wu, bu, wd, bd = [f(v) for v in golden_params(t)]
    x, dy = t["x"].float(), t["dy"].float()
    rows = x.numel() // x.shape[-1]
    ks = orc.keep_scale_tensor(rows, wg.shape[0], meta.get("dropout_p", 0.0), meta.get("seed", 0),
                               meta.get("offset", 0))
    act = meta.get("act", "silu")
    y = orc.forward(x, wg, bg, wu, bu, wd, bd, ks, act)
    torch.testing.assert_close(y, t["y"], rtol=1e-5, atol=1e-5)
    grads = orc.backward(x, wg, bg, wu, bu, wd, bd, dy, ks, act)
    for k, v in grads.items():
        torch.testing.assert_close(v, t[k], rtol=2e-5, atol=2e-5, msg=lambda m, k=k: f"{k}: {m}")
    expected = {k for k in t if k.startswith("d") and k != "dy"}
    assert set(grads) == expected


def test_oracle_matches_reference_ops():
    t, _, _ = load_golden("ops_closed_form_bf16")
    x, wu, wg, go = t["x"].float(), t["W_up"].float(), t["W_gp"].float(), t["grad_output"].float()
    h, g, u = orc.hidden_forward(x, wg, None, wu, None)
    torch.testing.assert_close(h, t["h"], rtol=1e-6, atol=1e-9)
    dx, dw_up, dw_gp, _, _ = orc.hidden_backward(x, wg, wu, g, u, go)
    for got, key in ((dx, "dx"), (dw_up, "dW_up"), (dw_gp, "dW_gp")):
        rel = ((got - t[key]).norm() / t[key].norm()).item()
        assert rel < 1e-6, (key, rel)  # the reference's own check is a relative Frobenius norm


def test_case_generator_is_deterministic_and_rounded():
    a = orc.make_case(8, 32, 48, True, torch.bfloat16, seed=3)
    b = orc.make_case(8, 32, 48, True, torch.bfloat16, seed=3)
    assert all(torch.equal(p, q) for p, q in zip(a.f32(), b.f32()))
    assert a.x.dtype == torch.bfloat16 and a.f32()[0].dtype == torch.float32
    c = orc.make_case(8, 32, 48, False, torch.float16, seed=3, w_std=None, x_dist="uniform")
    assert c.b_gate is None and c.x.min() >= 0 and c.w_gate.abs().max() <= 1 / 32 ** 0.5 + 1e-3


def test_parity_metric():
    want = torch.ones(10)
    assert orc.parity_errors(want + 0.01, want) == pytest.approx((0.01, 0.01), rel=1e-4)
    with pytest.raises(AssertionError):
        orc.assert_parity(want + 0.05, want, "t")
    # outputs with rms > 1: output rounding is not counted, the rest is measured in units of the rms
    big = torch.full((4,), 16.0)
    assert orc.parity_errors(big + 0.32, big) == pytest.approx((0.02, 0.02), rel=1e-4)
    orc.assert_parity((big + 0.125).to(torch.bfloat16), big, "next bf16 above 16")
    with pytest.raises(AssertionError):
        orc.assert_parity(big + 0.5, big, "too far")


def test_oracle_rmsnorm_matches_torch_rmsnorm_plus_reference_module():
    """Fixture norm_mlp_bf16: torch.nn.RMSNorm followed by the reference's EagerGatedMLP, through autograd."""
    t, meta, _ = load_golden("norm_mlp_bf16")
    f = lambda v: None if v is None else v.float()
    wg, bg, wu, bu, wd, bd = [f(v) for v in golden_params(t)]
    case = orc.Case(t["x"], t["p.gate_proj.weight"], t["p.gate_proj.bias"], t["p.up_proj.weight"],
                    t["p.up_proj.bias"], t["p.down_proj.weight"], t["p.down_proj.bias"], t["dy"])
    got = orc.norm_forward_backward(case, t["norm_weight"], float(meta["eps"]))
    for k, v in got.items():
        torch.testing.assert_close(v, t[k], rtol=3e-5, atol=3e-5, msg=lambda m, k=k: f"{k}: {m}")
    # and the norm alone against torch's module
    norm = torch.nn.RMSNorm(case.x.shape[-1], eps=float(meta["eps"]))
    with torch.no_grad():
        norm.weight.copy_(t["norm_weight"].float())
    torch.testing.assert_close(orc.rmsnorm(case.x.float(), t["norm_weight"].float(), float(meta["eps"])),
                               norm(case.x.float()), rtol=1e-6, atol=1e-6)
