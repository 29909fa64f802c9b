"""B200-native gated MLP: the reference's FusedGatedMLP API on hand-written sm_100a kernels.

The directory name carries a hyphen, so the package is imported under the name
`triton_gated_mlp_b200` through the thin directory of that name at the repository
root: with the root on sys.path,
`from triton_gated_mlp_b200.gated_mlp import FusedGatedMLP` is the one-line swap
for `from triton_gated_mlp.gated_mlp import FusedGatedMLP`.
"""
from . import _lib, build, host_pipeline, parallel  # noqa: F401
from .gated_mlp import FusedGatedMLP, FusedGatedMLPFunction, mlp_hidden_states_bwd, mlp_hidden_states_fwd  # noqa: F401

__all__ = [
    "FusedGatedMLP", "FusedGatedMLPFunction", "mlp_hidden_states_fwd", "mlp_hidden_states_bwd",
    "parallel", "build", "host_pipeline",
]
