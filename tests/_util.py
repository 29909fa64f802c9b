"""Shared helpers for the tests: golden-fixture loading and module construction."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"
DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def load_golden(name: str):
    """Returns (tensors, meta). 16-bit tensors were stored as raw bit patterns."""
    z = np.load(GOLDEN / f"{name}.npz")
    meta = {k[5:]: z[k].item() for k in z.files if k.startswith("meta.")}
    dt = DTYPES.get(meta.get("dtype", "bfloat16"), torch.bfloat16)
    out = {}
    for k in z.files:
        if k.startswith("meta."):
            continue
        a = z[k]
        if a.dtype == np.int16:
            out[k] = torch.from_numpy(a.copy()).view(dt)
        else:
            out[k] = torch.from_numpy(a.copy())
    return out, meta, dt


def golden_params(t):
    """(w_gate, b_gate, w_up, b_up, w_down, b_down) from a module fixture."""
    g = lambda k: t.get(k)
    return (g("p.gate_proj.weight"), g("p.gate_proj.bias"), g("p.up_proj.weight"), g("p.up_proj.bias"),
            g("p.down_proj.weight"), g("p.down_proj.bias"))


def build_module(pkg, case, dtype, device, dropout_p=0.0, **kw):
    """FusedGatedMLP loaded with a Case's weights, on `device` in `dtype`."""
    K, N = case.w_gate.shape[1], case.w_gate.shape[0]
    m = pkg.FusedGatedMLP(K, N, bias=case.b_gate is not None, dropout_p=dropout_p, **kw)
    m.load_state_dict(case.state_dict())
    return m.to(device).to(dtype)
