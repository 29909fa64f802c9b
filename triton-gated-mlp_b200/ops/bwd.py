"""Op-level backward with the reference's name and argument meaning.

Mirrors mlp_hidden_states_bwd of the reference
(src/triton_gated_mlp/ops/bwd.py:466-602): given x, the two [N, K] weights and
the gradient of the hidden state, returns (dx, dW_up, dW_gp). Like the
reference it recomputes the gate / up pre-activations from x (ops/bwd.py:180-193)
because this entry point receives no saved activations; the module-level
autograd function saves them instead and never calls this path. The weight
gradients sum over ALL token rows (the closed form the reference's own test
checks, tests/test_gated_mlp_bwd.py:108-123).
"""
from __future__ import annotations

from torch import Tensor

from . import kernels


def mlp_hidden_states_bwd(x: Tensor, W_up: Tensor, W_gp: Tensor, grad_output: Tensor):
    assert x.ndim == 2 and grad_output.ndim == 2, "x and grad_output must be 2-D"
    assert W_up.shape == W_gp.shape, "dimension mismatch in W_up or W_gp"
    assert W_up.shape[1] == x.shape[1], "dimension mismatch in W_up or x"
    assert grad_output.shape == (x.shape[0], W_up.shape[0]), "dimension mismatch in grad_output"
    if x.shape[1] % 16 != 0 or W_up.shape[0] % 16 != 0:
        raise NotImplementedError()
    _, g, u = kernels.hidden_fwd(x, W_gp, None, W_up, None, save=True)
    d_gate, d_up = kernels.bwd_dact(grad_output, g, u)
    dx = kernels.bwd_dx(d_gate, d_up, W_gp, W_up)
    dW_gp, dW_up = kernels.bwd_dw_gate_up(d_gate, d_up, x)[:2]
    return dx, dW_up, dW_gp
