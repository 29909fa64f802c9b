"""CPU restatement of the 8-bit (e4m3) decode path's quantisation contract.
TEST INFRASTRUCTURE ONLY (tests/, smoke, bench.py's checks): never imported by the package.

The reference has no low-precision path (its benchmark is fp16 only,
src/triton_gated_mlp/benchmark.py:26-123), so there is nothing of the reference to pin this to:
the format itself is pinned against known e4m3 values (tests/test_oracle_fp8.py), and the
arithmetic around it is the eager gated MLP of gated_mlp_oracle.py.

  weights      w8 = e4m3(W / ws[:, None]),  ws[r] = amax|W[r, :]| / 448      (once, per weight row)
  activations  a8 = e4m3(a / as[:, None]),  as[m] = max(amax|a[m, :]|, 1e-30) / 448   (per token, per call)
  products     (a8 * as) @ (w8 * ws)^T in fp32; the hidden state is rounded to the 16-bit
               format before it is quantised for the down projection, as the kernels store it.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import gated_mlp_oracle as orc

E4M3_MAX = 448.0


def e4m3_round(t: Tensor) -> Tensor:
    """fp32 values rounded to the nearest e4m3 value (ties to even), saturating at +-448."""
    return t.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()


def quantize_rows(a: Tensor):
    """(dequantised rows, scale) under the per-row contract above."""
    a = a.float()
    scale = a.abs().amax(dim=-1).clamp_min(1e-30) / E4M3_MAX
    return e4m3_round(a / scale[:, None]) * scale[:, None], scale


def dequantize_weight(w8: Tensor, scale: Tensor) -> Tensor:
    """fp32 weights from e4m3 bytes (uint8) and per-row scales."""
    return w8.view(torch.float8_e4m3fn).float() * scale.float()[:, None]


def decode_forward(x: Tensor, wg: Tensor, bg: Optional[Tensor], wu: Tensor, bu: Optional[Tensor], wd: Tensor,
                   bd: Optional[Tensor], hidden_dtype: torch.dtype = torch.bfloat16, act: str = "silu",
                   quantize_activations: bool = True) -> Tensor:
    """y of the 8-bit decode path for DEQUANTISED weights wg / wu / wd (fp32). With
    quantize_activations=False the activations stay as they are: what the same weights give without the
    activation quantisation (the reference point for the accuracy that costs)."""
    xq = quantize_rows(x)[0] if quantize_activations else x.float()
    h, _, _ = orc.hidden_forward(xq, wg, bg, wu, bu, None, act)
    h = h.to(hidden_dtype).float()
    hq = quantize_rows(h)[0] if quantize_activations else h
    y = hq @ wd.T
    return y if bd is None else y + bd
