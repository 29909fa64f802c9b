"""Generates the golden fixtures in this directory from the REFERENCE's own code.

Run in the build container, where the reference checkout is mounted read-only:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's torch-eager implementation unmodified
(src/triton_gated_mlp/gated_mlp.py: EagerGatedMLP :73-98, eager_fwd :105-128,
eager_bwd :131-156). The reference package imports `triton_dejavu` at module load
(ops/fwd.py:7, ops/bwd.py:8), which is not installable offline, so a stand-in
module with an identity `autotune` decorator is registered first; the Triton
kernels it would decorate are never called here.

The fixtures hold inputs (already rounded to the 16-bit dtype the engine runs in)
and the reference's fp32 CPU outputs, so tests on a machine without the reference
can pin both the CPU oracle and the CUDA kernels against them. For the dropout
fixture the reference module's nn.Dropout is replaced by a multiply with the
externally generated Philox mask (oracle/philox.py), because nn.Dropout's own mask
cannot be reproduced by another implementation.
"""
from __future__ import annotations

import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
from oracle import philox  # noqa: E402


def import_reference(ref_root: str):
    stub = types.ModuleType("triton_dejavu")

    def autotune(*a, **k):
        return lambda fn: fn

    class ConfigSpace:
        def __init__(self, *a, **k):
            pass

    stub.autotune = autotune
    stub.ConfigSpace = ConfigSpace
    sys.modules["triton_dejavu"] = stub
    sys.path.insert(0, str(Path(ref_root) / "src"))
    # import the submodule directly: the package __init__ pulls in tqdm-driven tooling
    import importlib
    return importlib.import_module("triton_gated_mlp.gated_mlp")


def rounded(t: torch.Tensor, dt: torch.dtype) -> torch.Tensor:
    return t.to(dt).float()


def np16(t: torch.Tensor, dt: torch.dtype) -> np.ndarray:
    """Store a 16-bit-rounded fp32 tensor as raw uint16 bit patterns (bf16 has no numpy dtype)."""
    return t.to(dt).view(torch.int16).numpy().copy()


def module_case(ref, name, K, N, bias, x_shape, dt, seed_w, seed_x, seed_dy, x_uniform, dy_std=1.0,
                dropout=None, hidden_act="silu"):
    torch.manual_seed(seed_w)
    m = ref.EagerGatedMLP(hidden_size=K, intermediate_size=N, bias=bias, dropout_p=0.0, hidden_act=hidden_act)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(rounded(p, dt))
    torch.manual_seed(seed_x)
    x = torch.rand(x_shape) if x_uniform else torch.randn(x_shape)
    x = rounded(x, dt).requires_grad_(True)
    torch.manual_seed(seed_dy)
    dy = rounded(torch.randn(x_shape) * dy_std, dt)
    meta = {"dtype": str(dt).split(".")[-1], "bias": bias, "act": hidden_act}
    if dropout is not None:
        p, seed, offset = dropout
        rows = x.numel() // K
        keep = philox.keep_mask(rows, N, p, seed, offset)
        ks = torch.from_numpy(keep.astype(np.float32) * philox.scale(p))

        class MaskDropout(torch.nn.Module):
            def forward(self, h):
                return h * ks

        m.dropout = MaskDropout()
        meta.update({"dropout_p": p, "seed": seed, "offset": offset})
    y = m(x)
    y.backward(dy)
    out = {
        "x": np16(x.detach(), dt), "dy": np16(dy, dt), "y": y.detach().numpy(), "dx": x.grad.numpy(),
    }
    for pname, p in m.named_parameters():
        out["p." + pname] = np16(p.detach(), dt)
        out["d" + pname] = p.grad.numpy()
    for k, v in meta.items():
        out["meta." + k] = np.array(v)
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, {k: v.shape for k, v in out.items() if hasattr(v, "shape") and v.ndim})


def norm_case(ref, name):
    """A Llama block's norm + MLP: torch.nn.RMSNorm followed by the reference's eager module, through autograd."""
    dt = torch.bfloat16
    K, N, M, eps = 128, 256, 72, 1e-5
    torch.manual_seed(60)
    m = ref.EagerGatedMLP(hidden_size=K, intermediate_size=N, bias=True, dropout_p=0.0)
    norm = torch.nn.RMSNorm(K, eps=eps)
    with torch.no_grad():
        norm.weight.copy_(rounded(1.0 + 0.2 * torch.randn(K), dt))
        for p in m.parameters():
            p.copy_(rounded(p, dt))
    torch.manual_seed(61)
    x = rounded(torch.randn((M, K)) * 1.7, dt).requires_grad_(True)
    torch.manual_seed(62)
    dy = rounded(torch.randn((M, K)) * 0.1, dt)
    y = m(norm(x))
    y.backward(dy)
    out = {"x": np16(x.detach(), dt), "dy": np16(dy, dt), "y": y.detach().numpy(), "dx": x.grad.numpy(),
           "norm_weight": np16(norm.weight.detach(), dt), "dinput_norm_weight": norm.weight.grad.numpy(),
           "meta.dtype": np.array("bfloat16"), "meta.eps": np.array(eps), "meta.bias": np.array(True)}
    for pname, p in m.named_parameters():
        out["p." + pname] = np16(p.detach(), dt)
        out["d" + pname] = p.grad.numpy()
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "ok")


def ops_case(ref, name):
    """The known-answer recipe of the reference's tests/test_gated_mlp_bwd.py:96-123 through its own
    eager_fwd / eager_bwd."""
    dt = torch.bfloat16
    B, M, N, K = 2, 32, 512, 256
    torch.manual_seed(5)
    x = rounded(torch.rand((B * M, K)) / K, dt)
    W_up = rounded(torch.rand((N, K)) / K, dt)
    W_gp = rounded(torch.rand((N, K)) / K, dt)
    grad_output = rounded(torch.rand((B * M, N)) / K, dt)
    h = ref.eager_fwd(x, W_up, None, W_gp, None)
    dx, dW_up, dW_gp = ref.eager_bwd(x, W_up, W_gp, grad_output)
    np.savez_compressed(
        HERE / f"{name}.npz", x=np16(x, dt), W_up=np16(W_up, dt), W_gp=np16(W_gp, dt),
        grad_output=np16(grad_output, dt), h=h.numpy(), dx=dx.numpy(), dW_up=dW_up.numpy(), dW_gp=dW_gp.numpy(),
    )
    print(name, "ok")


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref = import_reference(sys.argv[1])
    # README / benchmark configuration 1: M=128, K=512, N=256, no bias, fp16 engine.
    module_case(ref, "c1_readme_fp16", K=512, N=256, bias=False, x_shape=(128, 512), dt=torch.float16,
                seed_w=0, seed_x=0, seed_dy=1, x_uniform=True)
    # Default constructor (K=256, N=512, bias=True) on a 3-D input, like tests/test_gated_mlp_bwd.py:37-41.
    module_case(ref, "default_bias_3d_bf16", K=256, N=512, bias=True, x_shape=(4, 24, 256), dt=torch.bfloat16,
                seed_w=10, seed_x=11, seed_dy=12, x_uniform=True, dy_std=0.1)
    # Bias + dropout with the externally supplied Philox mask; ragged M (not a multiple of the tile).
    module_case(ref, "dropout_bias_bf16", K=128, N=384, bias=True, x_shape=(200, 128), dt=torch.bfloat16,
                seed_w=20, seed_x=21, seed_dy=22, x_uniform=False, dy_std=0.1, dropout=(0.1, 0x5EED, 7))
    # The other gate activations of the reference's ACT_FWD table, through its eager module and
    # torch autograd (small shapes; one fixture per activation).
    for i, act in enumerate(("gelu", "relu", "sigmoid", "tanh", "leaky_relu", "no_act")):
        module_case(ref, f"act_{act}_bf16", K=64, N=128, bias=True, x_shape=(40, 64), dt=torch.bfloat16,
                    seed_w=30 + i, seed_x=40 + i, seed_dy=50 + i, x_uniform=False, dy_std=0.1, hidden_act=act)
    ops_case(ref, "ops_closed_form_bf16")
    norm_case(ref, "norm_mlp_bf16")


if __name__ == "__main__":
    main()
