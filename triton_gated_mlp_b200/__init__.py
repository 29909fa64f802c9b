"""Importable name of the package that lives in ../triton-gated-mlp_b200 (a directory name with a hyphen
cannot be imported). With the repository root on sys.path,

    from triton_gated_mlp_b200.gated_mlp import FusedGatedMLP

is the one-line swap for `from triton_gated_mlp.gated_mlp import FusedGatedMLP`. This file holds no code of
its own: it points the package's search path at that directory and runs its __init__.
"""
from pathlib import Path as _Path

_real = _Path(__file__).resolve().parent.parent / "triton-gated-mlp_b200"
__path__ = [str(_real)]
exec(compile((_real / "__init__.py").read_text(), str(_real / "__init__.py"), "exec"))
