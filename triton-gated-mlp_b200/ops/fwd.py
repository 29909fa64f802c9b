"""Op-level forward with the reference's name and argument meaning.

Mirrors mlp_hidden_states_fwd of the reference
(src/triton_gated_mlp/ops/fwd.py:198-279): same positional arguments, same
preconditions and exception types (validate_dimensions, :169-184; the K % 16 /
N % 16 NotImplementedError, :224-230), but bias and dropout are honoured
instead of being dropped, as EagerGatedMLP does (gated_mlp.py:96).
"""
from __future__ import annotations

from typing import Optional

from torch import Tensor

from . import kernels
from .kernels import Dropout, Shard, NO_SHARD

from .._lib import ACT_CODES

# The reference's module accepts these names (gated_mlp.py:27-37); its own fused kernel
# implements only "silu" and "no_act" (ops/act.py:7-12).
SUPPORTED_ACTS = tuple(ACT_CODES)


def validate_dimensions(x: Tensor, WT_up: Tensor, b_up: Optional[Tensor], WT_gp: Tensor,
                        b_gp: Optional[Tensor]) -> None:
    assert x.ndim <= 2, f"input tensor must have ndims <=2, got {x.ndim}"
    assert WT_up.shape[1] == x.shape[1], "dimension mismatch in WT_up or x"
    assert WT_gp.shape == WT_up.shape, "dimension mismatch in WT_up or WT_gp"
    if b_up is not None:
        assert b_up.shape[0] == WT_up.shape[0], "dimension mismatch in b_up"
    if b_gp is not None:
        assert b_gp.shape[0] == WT_up.shape[0], "dimension mismatch in b_gp"


def mlp_hidden_states_fwd(
    x: Tensor,
    WT_up: Tensor,
    b_up: Optional[Tensor],
    WT_gp: Tensor,
    b_gp: Optional[Tensor],
    act_fn: str = "silu",
    dropout_p: float = 0.0,
    *,
    seed: int = 0,
    offset: int = 0,
    shard: Shard = NO_SHARD,
    save_preact: bool = False,
):
    """dropout(act_fn(x @ WT_gp.T + b_gp) * (x @ WT_up.T + b_up)) in one tcgen05 kernel.

    Weights are nn.Linear-shaped ([N, K]). With save_preact=True returns
    (H, G, U) where G and U are the biased gate / up pre-activations.
    """
    validate_dimensions(x, WT_up, b_up, WT_gp, b_gp)
    if act_fn not in SUPPORTED_ACTS:
        raise NotImplementedError(f"gate activation {act_fn!r}: supported are {sorted(SUPPORTED_ACTS)}")
    K = x.shape[1]
    N = WT_up.shape[0]
    if K % 16 != 0:
        raise NotImplementedError()
    if N % 16 != 0:
        raise NotImplementedError()
    drop = Dropout(float(dropout_p), seed, offset)
    return kernels.hidden_fwd(x, WT_gp, b_gp, WT_up, b_up, drop=drop, shard=shard, save=save_preact, act=act_fn)
