"""CPU restatement (torch fp32 on the host) of the reference's eager gated MLP.
TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and
bench.py's CPU baseline legs, never by the shipped package.

What it restates (paths relative to the reference project):
  forward    EagerGatedMLP.forward, src/triton_gated_mlp/gated_mlp.py:92-98:
             y = down(dropout(silu(gate(x)) * up(x))), bias on all three linears.
  backward   the closed form of eager_bwd (gated_mlp.py:131-156; the same block is
             the known-answer recipe of tests/test_gated_mlp_bwd.py:108-123),
             extended by the down projection's and the biases' gradients, which
             the reference leaves to torch autograd.
  silu'      _silu_op_bwd, gated_mlp.py:40-43.
Dropout uses the counter-based mask of oracle/philox.py instead of nn.Dropout's
generator (see that file for why).

Pinned by tests/test_oracle_golden.py against outputs of the reference's own
EagerGatedMLP / eager_fwd / eager_bwd, generated in the build container by
tests/golden/make_golden.py (the reference publishes no golden vectors).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import numpy as np
import torch
from torch import Tensor

from . import philox

# Tolerances of the parity contract for 16-bit kernels against this fp32 oracle.
MAX_ABS_TOL = 2e-2
MEAN_REL_TOL = 1e-2


# ------------------------------------------------------------------ math ----
def silu(b: Tensor) -> Tensor:
    return b * torch.sigmoid(b)


def silu_prime(b: Tensor) -> Tensor:
    """sigma * (1 + b * (1 - sigma)), gated_mlp.py:41-42."""
    sigma = 1 / (1 + torch.exp(-b))
    return sigma * (1 + b * (1 - sigma))


# Gate activations by the names of the reference's ACT_FWD table (gated_mlp.py:27-37): value and
# derivative. The reference defines a derivative for SiLU only (ACT_BWD, gated_mlp.py:46-55); the
# others are the textbook forms of the torch modules that table holds (nn.GELU is the erf form,
# nn.LeakyReLU has slope 0.01).
def act_value(name: str, b: Tensor) -> Tensor:
    if name in ("silu", "swish"):
        return silu(b)
    if name == "no_act":
        return b
    if name == "relu":
        return torch.relu(b)
    if name == "gelu":
        return 0.5 * b * (1 + torch.erf(b / 2 ** 0.5))
    if name == "sigmoid":
        return torch.sigmoid(b)
    if name == "tanh":
        return torch.tanh(b)
    if name == "leaky_relu":
        return torch.where(b > 0, b, 0.01 * b)
    raise NotImplementedError(name)


def act_prime(name: str, b: Tensor) -> Tensor:
    if name in ("silu", "swish"):
        return silu_prime(b)
    if name == "no_act":
        return torch.ones_like(b)
    if name == "relu":
        return (b > 0).to(b.dtype)
    if name == "gelu":
        return 0.5 * (1 + torch.erf(b / 2 ** 0.5)) + b * torch.exp(-0.5 * b * b) / (2 * torch.pi) ** 0.5
    if name == "sigmoid":
        s = torch.sigmoid(b)
        return s * (1 - s)
    if name == "tanh":
        return 1 - torch.tanh(b) ** 2
    if name == "leaky_relu":
        return torch.where(b > 0, torch.ones_like(b), torch.full_like(b, 0.01))
    raise NotImplementedError(name)


def hidden_forward(x, w_gate, b_gate, w_up, b_up, keep_scale: Optional[Tensor] = None, act: str = "silu"):
    """(H, G, U): hidden state after dropout and the biased pre-activations."""
    g = x @ w_gate.T
    if b_gate is not None:
        g = g + b_gate
    u = x @ w_up.T
    if b_up is not None:
        u = u + b_up
    h = act_value(act, g) * u
    if keep_scale is not None:
        h = h * keep_scale
    return h, g, u


def forward(x, w_gate, b_gate, w_up, b_up, w_down, b_down, keep_scale: Optional[Tensor] = None,
            act: str = "silu") -> Tensor:
    shapes = x.shape
    x2 = x.reshape(-1, shapes[-1])
    h, _, _ = hidden_forward(x2, w_gate, b_gate, w_up, b_up, keep_scale, act)
    y = h @ w_down.T
    if b_down is not None:
        y = y + b_down
    return y.reshape(shapes[:-1] + (w_down.shape[0],))


def hidden_backward(x, w_gate, w_up, g, u, dh, act: str = "silu"):
    """(dx, dW_up, dW_gate, d_gate, d_up) from dH; eager_bwd's closed form, gated_mlp.py:143-154."""
    c = act_value(act, g)
    d_gate = (dh * u) * act_prime(act, g)   # grad_output_a_act_prime
    d_up = dh * c                       # grad_output_c
    dx = d_up @ w_up + d_gate @ w_gate
    return dx, d_up.T @ x, d_gate.T @ x, d_gate, d_up


def backward(x, w_gate, b_gate, w_up, b_up, w_down, b_down, dy, keep_scale: Optional[Tensor] = None,
             act: str = "silu") -> Dict[str, Tensor]:
    """All gradients of forward() for upstream gradient dy. Keys follow nn.Module parameter names."""
    x2 = x.reshape(-1, x.shape[-1])
    dy2 = dy.reshape(-1, dy.shape[-1])
    h, g, u = hidden_forward(x2, w_gate, b_gate, w_up, b_up, keep_scale, act)
    dh = dy2 @ w_down
    if keep_scale is not None:
        dh = dh * keep_scale
    dx, dw_up, dw_gate, d_gate, d_up = hidden_backward(x2, w_gate, w_up, g, u, dh, act)
    out = {
        "dx": dx.reshape(x.shape),
        "dgate_proj.weight": dw_gate,
        "dup_proj.weight": dw_up,
        "ddown_proj.weight": dy2.T @ h,
    }
    if b_gate is not None:
        out["dgate_proj.bias"] = d_gate.sum(0)
    if b_up is not None:
        out["dup_proj.bias"] = d_up.sum(0)
    if b_down is not None:
        out["ddown_proj.bias"] = dy2.sum(0)
    return out


# -------------------------------------------------------------- RMSNorm ----
# The step before the MLP in a Llama block. The reference has no norm; the definition
# restated here is torch.nn.RMSNorm's: x * rsqrt(mean(x^2, -1) + eps) * weight. Pinned by the
# fixture norm_mlp_bf16 (torch.nn.RMSNorm followed by the reference's EagerGatedMLP).
def rmsnorm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rmsnorm_backward(x: Tensor, weight: Tensor, eps: float, dout: Tensor):
    """(dx, dweight) of rmsnorm for upstream gradient dout (closed form)."""
    rs = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    xn = x * rs
    dxn = dout * weight
    dx = rs * (dxn - xn * (dxn * xn).mean(-1, keepdim=True))
    return dx, (dout * xn).reshape(-1, x.shape[-1]).sum(0)


def norm_forward_backward(case: "Case", norm_weight: Tensor, eps: float) -> Dict[str, Tensor]:
    """fp32 oracle outputs of y = MLP(rmsnorm(x)): {"y", "dx", "dinput_norm_weight", "dgate_proj.weight", ...}."""
    x, wg, bg, wu, bu, wd, bd, dy = case.f32()
    w = norm_weight.float()
    xn = rmsnorm(x, w, eps)
    out = {"y": forward(xn, wg, bg, wu, bu, wd, bd)}
    grads = backward(xn, wg, bg, wu, bu, wd, bd, dy)
    dx, dw = rmsnorm_backward(x, w, eps, grads.pop("dx"))
    out.update(grads)
    out["dx"], out["dinput_norm_weight"] = dx, dw
    return out


def keep_scale_tensor(rows: int, cols: int, p: float, seed: int, offset: int, *, row0: int = 0,
                      col0: int = 0, n_global: Optional[int] = None) -> Optional[Tensor]:
    """mask * 1/(1-p) as fp32, or None when p == 0."""
    if p <= 0.0:
        return None
    keep = philox.keep_mask(rows, cols, p, seed, offset, row0=row0, col0=col0, n_global=n_global)
    return torch.from_numpy(keep.astype(np.float32) * philox.scale(p))


# ----------------------------------------------------------------- cases ----
@dataclass
class Case:
    """Seeded inputs of one configuration, already rounded to the engine's dtype.

    The tensors are stored in the low-precision dtype; the oracle up-casts them to
    fp32, so a comparison measures kernel error, not input quantisation.
    """

    x: Tensor
    w_gate: Tensor
    b_gate: Optional[Tensor]
    w_up: Tensor
    b_up: Optional[Tensor]
    w_down: Tensor
    b_down: Optional[Tensor]
    dy: Tensor

    def state_dict(self) -> Dict[str, Tensor]:
        sd = {"gate_proj.weight": self.w_gate, "up_proj.weight": self.w_up, "down_proj.weight": self.w_down}
        if self.b_gate is not None:
            sd.update({"gate_proj.bias": self.b_gate, "up_proj.bias": self.b_up, "down_proj.bias": self.b_down})
        return {k: v.float() for k, v in sd.items()}

    def f32(self):
        f = lambda t: None if t is None else t.float()
        return (f(self.x), f(self.w_gate), f(self.b_gate), f(self.w_up), f(self.b_up), f(self.w_down),
                f(self.b_down), f(self.dy))


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def make_case(M: int, K: int, N: int, bias: bool, dtype: torch.dtype, seed: int = 0, x_dist: str = "normal",
              w_std: Optional[float] = 0.02, dy_std: float = 1.0, b_std: float = 0.02,
              lead_shape: Optional[tuple] = None) -> Case:
    """Synthetic inputs with the value distributions the benchmark configurations name.

    One generator per tensor, seeded seed + tensor index, drawn in fp32 on the CPU and
    then rounded to `dtype`. w_std=None draws nn.Linear's default init
    (uniform(-1/sqrt(fan_in), 1/sqrt(fan_in))).
    """
    def normal(shape, std, idx):
        return (torch.randn(shape, generator=_gen(seed + idx)) * std).to(dtype)

    def linear_default(shape, idx):
        bound = 1.0 / (shape[1] ** 0.5)
        return ((torch.rand(shape, generator=_gen(seed + idx)) * 2 - 1) * bound).to(dtype)

    xs = (M, K) if lead_shape is None else tuple(lead_shape) + (K,)
    if x_dist == "uniform":
        x = torch.rand(xs, generator=_gen(seed)).to(dtype)
    else:
        x = torch.randn(xs, generator=_gen(seed)).to(dtype)
    if w_std is None:
        w_gate, w_up, w_down = linear_default((N, K), 1), linear_default((N, K), 2), linear_default((K, N), 3)
    else:
        w_gate, w_up, w_down = normal((N, K), w_std, 1), normal((N, K), w_std, 2), normal((K, N), w_std, 3)
    b_gate = normal((N,), b_std, 4) if bias else None
    b_up = normal((N,), b_std, 5) if bias else None
    b_down = normal((K,), b_std, 6) if bias else None
    dy = (torch.randn(xs, generator=_gen(seed + 7)) * dy_std).to(dtype)
    return Case(x, w_gate, b_gate, w_up, b_up, w_down, b_down, dy)


def forward_backward(case: Case, dropout_p: float = 0.0, seed: int = 0, offset: int = 0, *, row0: int = 0,
                     col0: int = 0, n_global: Optional[int] = None, grads: bool = True,
                     act: str = "silu") -> Dict[str, Tensor]:
    """fp32 oracle outputs for a case: {"y", "dx", "dgate_proj.weight", ...}."""
    x, wg, bg, wu, bu, wd, bd, dy = case.f32()
    rows = x.numel() // x.shape[-1]
    ks = keep_scale_tensor(rows, wg.shape[0], dropout_p, seed, offset, row0=row0, col0=col0, n_global=n_global)
    out = {"y": forward(x, wg, bg, wu, bu, wd, bd, ks, act)}
    if grads:
        out.update(backward(x, wg, bg, wu, bu, wd, bd, dy, ks, act))
    return out


# ---------------------------------------------------------------- parity ----
# Largest relative error of rounding an exact value to the 16-bit output format.
HALF_ULP_REL = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11}


def parity_errors(got: Tensor, want: Tensor, half_ulp_rel: float = 0.0):
    """(max abs error, mean relative error) in the sense of the parity contract.

    max abs error  = max(|got - want| - half_ulp_rel * |want|, 0) / max(1, rms(want)).
    The contract's absolute bound is meant for outputs of order one. At the benchmark
    configurations' own distributions outputs are larger (decode: rms(y) = 4.4, |y| up to
    20, where neighbouring bf16 values are 0.125 apart), so (a) the error that rounding
    the exact result to the output format would make anyway is not counted, and (b) the
    rest is measured in units of the output's rms when that exceeds one. For outputs of
    order one and half_ulp_rel = 0 this is the plain max abs error.
    mean rel error = mean|got - want| / mean|want|.
    """
    got, want = got.double(), want.double()
    diff = (got - want).abs()
    excess = (diff - half_ulp_rel * want.abs()).clamp_min(0.0)
    scale = max(1.0, want.pow(2).mean().sqrt().item())
    denom = want.abs().mean().clamp_min(1e-30)
    return excess.max().item() / scale, (diff.mean() / denom).item()


def parity_report(got: Tensor, want: Tensor, out_dtype: torch.dtype = torch.bfloat16) -> Dict[str, float]:
    """Every figure of one comparison: the literal max abs error, the contract's figure
    (parity_errors), the mean relative error, and the scale of the expected values."""
    got, want = got.double(), want.double()
    scaled, mean_rel = parity_errors(got, want, HALF_ULP_REL[out_dtype])
    return {"max_abs": (got - want).abs().max().item(), "max_abs_scaled": scaled, "mean_rel": mean_rel,
            "rms_want": want.pow(2).mean().sqrt().item(), "max_want": want.abs().max().item()}


# Where the expected values are of order one (rms <= 1) and small enough that rounding them to
# the 16-bit output format cannot by itself use up much of the bound (|want| <= 2: at most
# 2**-8 * 2 = 0.008 in bf16), the LITERAL max abs error is held to the bound. Elsewhere the
# contract's figure applies (rounding of the output not counted, units of the output's rms).
LITERAL_MAX_WANT = 2.0


def assert_parity(got: Tensor, want: Tensor, name: str = "", max_abs: float = MAX_ABS_TOL,
                  mean_rel: float = MEAN_REL_TOL, out_dtype: Optional[torch.dtype] = None,
                  report: Optional[list] = None) -> None:
    """Parity contract for a 16-bit kernel output `got` against the fp32 oracle `want`.

    out_dtype: the kernel's output format (default: got.dtype when it is 16-bit, else bf16).
    report: a list that receives (name, parity_report) for callers that print the figures.
    """
    assert got.shape == want.shape, f"{name}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    if out_dtype is None:
        out_dtype = got.dtype if got.dtype in HALF_ULP_REL else torch.bfloat16
    got = got.float()
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    r = parity_report(got, want, out_dtype)
    if report is not None:
        report.append((name, r))
    literal = r["rms_want"] <= 1.0 and r["max_want"] <= LITERAL_MAX_WANT
    ma = r["max_abs"] if literal else r["max_abs_scaled"]
    assert ma <= max_abs and r["mean_rel"] <= mean_rel, (
        f"{name}: max abs err {ma:.3e} ({'literal' if literal else 'scaled'}; literal {r['max_abs']:.3e}, scaled "
        f"{r['max_abs_scaled']:.3e}, tol {max_abs:.1e}), mean rel err {r['mean_rel']:.3e} (tol {mean_rel:.1e}), "
        f"rms(want) {r['rms_want']:.3g}, max|want| {r['max_want']:.3g}"
    )
