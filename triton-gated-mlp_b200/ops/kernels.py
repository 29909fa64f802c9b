"""One Python function per libgmlp entry point: tensors in, tensors out.

These wrappers allocate outputs with torch (caller-owned device memory), check
what the C ABI cannot see (contiguity, dtype agreement, device), and enqueue the
kernel on torch's current stream. They never compute anything themselves.
"""
from __future__ import annotations

import contextlib
import ctypes as C
from dataclasses import dataclass

import torch
from torch import Tensor

from .. import _lib
from .._lib import ACT_CODES, Problem, check, dtype_code, load, ptr, require_cuda, stream_of


@dataclass(frozen=True)
class Dropout:
    """Dropout settings of one call: probability plus the Philox (seed, offset)."""

    p: float = 0.0
    seed: int = 0
    offset: int = 0


@dataclass(frozen=True)
class Shard:
    """Where this rank's rows / intermediate columns sit in the un-sharded problem."""

    row0: int = 0        # global index of local token row 0
    col0: int = 0        # global index of local intermediate column 0
    n_global: int = 0    # un-sharded intermediate size (0: same as local N)


NO_DROPOUT = Dropout()
NO_SHARD = Shard()


_SAME_DEVICE = contextlib.nullcontext()


def _on(dev: torch.device):
    """Context that makes `dev` current for a library call; free when it already is."""
    return _SAME_DEVICE if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)


def act_code(act: str) -> int:
    """gmlp_act_t for one of the reference's activation names; NotImplementedError otherwise."""
    if act not in ACT_CODES:
        raise NotImplementedError(f"gate activation {act!r}: supported are {sorted(ACT_CODES)}")
    return ACT_CODES[act]


def _problem(M: int, K: int, N: int, dt: torch.dtype, drop: Dropout, shard: Shard, act: str = "silu",
             tuning: int = 0) -> Problem:
    return Problem(
        M=M, K=K, N=N, dtype=dtype_code(dt), dropout_p=float(drop.p),
        seed=int(drop.seed) & 0xFFFFFFFFFFFFFFFF, offset=int(drop.offset) & 0xFFFFFFFFFFFFFFFF,
        row0_global=shard.row0, col0_global=shard.col0, N_global=shard.n_global, act=act_code(act),
        tuning=int(tuning),
    )


def _c(t: Tensor | None) -> Tensor | None:
    """Contiguous view of t (copies only if t is strided)."""
    return None if t is None else (t if t.is_contiguous() else t.contiguous())


def _same_dtype(*ts: Tensor | None) -> torch.dtype:
    dt = None
    for t in ts:
        if t is None:
            continue
        if dt is None:
            dt = t.dtype
        elif t.dtype != dt:
            raise TypeError(f"mixed dtypes: {dt} and {t.dtype}")
    return dt


def hidden_fwd(x: Tensor, w_gate: Tensor, b_gate: Tensor | None, w_up: Tensor, b_up: Tensor | None,
               drop: Dropout = NO_DROPOUT, shard: Shard = NO_SHARD, save: bool = False, act: str = "silu",
               tuning: int = 0, row_scale: Tensor | None = None):
    """H = dropout(act(x W_gate^T + b_gate) * (x W_up^T + b_up)); with save=True also
    returns the biased pre-activations (G, U). `tuning`: _lib.tune_word() for this launch.
    row_scale: optional fp32 [M] factors on both products before the bias (rms_rowscale's output)."""
    dev = require_cuda(x, w_gate, b_gate, w_up, b_up)
    dt = _same_dtype(x, w_gate, b_gate, w_up, b_up)
    x, w_gate, w_up, b_gate, b_up = _c(x), _c(w_gate), _c(w_up), _c(b_gate), _c(b_up)
    M, K = x.shape
    N = w_gate.shape[0]
    h = torch.empty((M, N), dtype=dt, device=dev)
    g = torch.empty((M, N), dtype=dt, device=dev) if save else None
    u = torch.empty((M, N), dtype=dt, device=dev) if save else None
    if M > 0:
        prob = _problem(M, K, N, dt, drop, shard, act, tuning)
        _check_row_scale(row_scale, M, dev)
        with _on(dev):
            check(load().gmlp_hidden_fwd_scaled(C.byref(prob), ptr(x), ptr(row_scale), ptr(w_gate), ptr(b_gate),
                                                ptr(w_up), ptr(b_up), ptr(h), ptr(g), ptr(u), stream_of(x)))
    return (h, g, u) if save else h


def _check_row_scale(rs: Tensor | None, M: int, dev: torch.device) -> None:
    if rs is not None and (rs.dtype != torch.float32 or rs.shape != (M,) or rs.device != dev
                           or not rs.is_contiguous()):
        raise ValueError(f"row_scale must be a contiguous float32 tensor of shape ({M},) on {dev}")


def rms_rowscale(x: Tensor, eps: float, normalised: bool = False):
    """rs[m] = 1 / sqrt(mean_k x[m,k]^2 + eps) as fp32 [M]; with normalised=True also x * rs[:, None] in
    x's dtype (what the backward pass of the norm needs)."""
    dev = require_cuda(x)
    x = _c(x)
    M, K = x.shape
    rs = torch.empty((M,), dtype=torch.float32, device=dev)
    xn = torch.empty((M, K), dtype=x.dtype, device=dev) if normalised else None
    if M > 0:
        with _on(dev):
            check(load().gmlp_rms_rowscale(M, K, dtype_code(x.dtype), ptr(x), x.stride(0), float(eps), ptr(rs),
                                           ptr(xn), stream_of(x)))
    return (rs, xn) if normalised else rs


def rms_bwd(dxn: Tensor, xn: Tensor, rs: Tensor) -> Tensor:
    """Backward of xn = x * rs[:, None]: dx = rs * (dxn - xn * mean_k(dxn * xn))."""
    dev = require_cuda(dxn, xn, rs)
    dt = _same_dtype(dxn, xn)
    dxn, xn = _c(dxn), _c(xn)
    M, K = dxn.shape
    _check_row_scale(rs, M, dev)
    dx = torch.empty((M, K), dtype=dt, device=dev)
    if M > 0:
        with _on(dev):
            check(load().gmlp_rms_bwd(M, K, dtype_code(dt), ptr(dxn), ptr(xn), ptr(rs), ptr(dx), stream_of(dxn)))
    return dx


def _out_buffer(out: Tensor | None, shape, dt: torch.dtype, dev: torch.device) -> Tensor:
    if out is None:
        return torch.empty(shape, dtype=dt, device=dev)
    if tuple(out.shape) != tuple(shape) or out.dtype != dt or out.device != dev or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous {tuple(shape)} {dt} tensor on {dev}")
    return out


def down_fwd(h: Tensor, w_down: Tensor, b_down: Tensor | None, residual: Tensor | None = None,
             out: Tensor | None = None, tuning: int = 0) -> Tensor:
    """y = h W_down^T (+ b_down) (+ residual), written into `out` when given."""
    dev = require_cuda(h, w_down, b_down, residual)
    dt = _same_dtype(h, w_down, b_down, residual)
    h, w_down, b_down, residual = _c(h), _c(w_down), _c(b_down), _c(residual)
    M, N = h.shape
    K = w_down.shape[0]
    y = _out_buffer(out, (M, K), dt, dev)
    if M > 0:
        prob = _problem(M, K, N, dt, NO_DROPOUT, NO_SHARD, tuning=tuning)
        with _on(dev):
            check(load().gmlp_down_fwd(C.byref(prob), ptr(h), ptr(w_down), ptr(b_down), ptr(residual),
                                       ptr(y), stream_of(h)))
    return y


def mlp_fwd(x: Tensor, w_gate: Tensor, b_gate: Tensor | None, w_up: Tensor, b_up: Tensor | None, w_down: Tensor,
            b_down: Tensor | None, drop: Dropout = NO_DROPOUT, shard: Shard = NO_SHARD, save: bool = False,
            act: str = "silu", residual: Tensor | None = None, tuning: int = 0):
    """The whole forward pass in one library call: (y, h, g, u) with g = u = None unless save=True."""
    dev = require_cuda(x, w_gate, b_gate, w_up, b_up, w_down, b_down, residual)
    dt = _same_dtype(x, w_gate, b_gate, w_up, b_up, w_down, b_down, residual)
    x, w_gate, w_up, w_down = _c(x), _c(w_gate), _c(w_up), _c(w_down)
    b_gate, b_up, b_down, residual = _c(b_gate), _c(b_up), _c(b_down), _c(residual)
    M, K = x.shape
    N = w_gate.shape[0]
    h = torch.empty((M, N), dtype=dt, device=dev)
    g = torch.empty((M, N), dtype=dt, device=dev) if save else None
    u = torch.empty((M, N), dtype=dt, device=dev) if save else None
    y = torch.empty((M, K), dtype=dt, device=dev)
    if M > 0:
        prob = _problem(M, K, N, dt, drop, shard, act, tuning)
        with _on(dev):
            check(load().gmlp_mlp_fwd(C.byref(prob), ptr(x), ptr(w_gate), ptr(b_gate), ptr(w_up), ptr(b_up),
                                      ptr(w_down), ptr(b_down), ptr(residual), ptr(h), ptr(g), ptr(u), ptr(y),
                                      stream_of(x)))
    return y, h, g, u


def mlp_bwd(dy: Tensor, x: Tensor, w_gate: Tensor, w_up: Tensor, w_down: Tensor, g: Tensor, u: Tensor, h: Tensor,
            drop: Dropout = NO_DROPOUT, shard: Shard = NO_SHARD, act: str = "silu", want_dx: bool = True,
            want_dw_gate_up: bool = True, want_dw_down: bool = True, want_db_gate: bool = False,
            want_db_up: bool = False, want_db_down: bool = False, inplace: bool = False, tuning: int = 0):
    """The whole backward pass in one library call. Returns a dict with the gradients asked for
    ("dx", "dw_gate", "dw_up", "dw_down", "db_gate", "db_up", "db_down") and "d_gate" / "d_up" when they were
    computed. Bias gradients come out of the weight-gradient kernels, so want_db_gate / want_db_up need
    want_dw_gate_up and want_db_down needs want_dw_down. inplace=True writes d_gate / d_up over g / u."""
    dev = require_cuda(dy, x, w_gate, w_up, w_down, g, u, h)
    dt = _same_dtype(dy, x, w_gate, w_up, w_down, g, u, h)
    if (want_db_gate or want_db_up) and not want_dw_gate_up or (want_db_down and not want_dw_down):
        raise ValueError("bias gradients are produced by the weight-gradient kernels: ask for those too")
    if dt == torch.float32:
        # fp32 path: the pass composed of the per-kernel calls above (each of them tf32 GEMMs on K-major copies)
        out = {}
        if want_dx or want_dw_gate_up:
            out["d_gate"], out["d_up"] = bwd_dhidden(dy, w_down, g, u, drop=drop, shard=shard, act=act)
        if want_dx:
            out["dx"] = bwd_dx(out["d_gate"], out["d_up"], w_gate, w_up)
        if want_dw_gate_up:
            r = bwd_dw_gate_up(out["d_gate"], out["d_up"], x, bias_grads=want_db_gate or want_db_up)
            out["dw_gate"], out["dw_up"] = r[0], r[1]
            if want_db_gate:
                out["db_gate"] = r[2]
            if want_db_up:
                out["db_up"] = r[3]
        if want_dw_down:
            r = bwd_dw_down(dy, h, bias_grad=want_db_down)
            out["dw_down"] = r[0] if want_db_down else r
            if want_db_down:
                out["db_down"] = r[1]
        return out
    if inplace and not (g.is_contiguous() and u.is_contiguous()):
        raise ValueError("inplace=True needs contiguous g and u")
    dy, x, w_gate, w_up, w_down, g, u, h = (_c(t) for t in (dy, x, w_gate, w_up, w_down, g, u, h))
    M, K = dy.shape
    N = w_down.shape[1]
    new = lambda *shape: torch.empty(shape, dtype=dt, device=dev)
    out = {}
    hidden = want_dx or want_dw_gate_up
    if hidden:
        out["d_gate"] = g if inplace else new(M, N)
        out["d_up"] = u if inplace else new(M, N)
    if want_dx:
        out["dx"] = new(M, K)
    if want_dw_gate_up:
        out["dw_gate"], out["dw_up"] = new(N, K), new(N, K)
    if want_dw_down:
        out["dw_down"] = new(K, N)
    if want_db_gate:
        out["db_gate"] = new(N)
    if want_db_up:
        out["db_up"] = new(N)
    if want_db_down:
        out["db_down"] = new(K)
    if M == 0:
        for k_, t in out.items():
            if k_ not in ("d_gate", "d_up"):
                t.zero_()
        return out
    prob = _problem(M, K, N, dt, drop, shard, act, tuning)
    o = out.get
    with _on(dev):
        scratch = bias_grad_scratch(K, N, dt, dev) if (want_db_gate or want_db_up or want_db_down) else None
        check(load().gmlp_mlp_bwd(
            C.byref(prob), ptr(dy), ptr(x), ptr(w_gate), ptr(w_up), ptr(w_down), ptr(g), ptr(u), ptr(h),
            ptr(o("d_gate")), ptr(o("d_up")), ptr(o("dx")), ptr(o("dw_gate")), ptr(o("dw_up")), ptr(o("dw_down")),
            ptr(o("db_gate")), ptr(o("db_up")), ptr(o("db_down")), ptr(scratch),
            0 if scratch is None else scratch.numel() * scratch.element_size(), stream_of(dy)))
    return out


def bwd_dhidden(dy: Tensor, w_down: Tensor, g: Tensor, u: Tensor, drop: Dropout = NO_DROPOUT,
                shard: Shard = NO_SHARD, act: str = "silu", inplace: bool = False, tuning: int = 0):
    """(d_gate, d_up) from dy through W_down and the activation/multiply derivative.

    inplace=True writes d_gate over g and d_up over u (both must be contiguous) and returns
    those tensors: two [M, N] buffers fewer, and the pre-activations are gone afterwards."""
    dev = require_cuda(dy, w_down, g, u)
    dt = _same_dtype(dy, w_down, g, u)
    if dt == torch.float32:
        # fp32 path: dH by the K-major tf32 GEMM (W_down transposed once), then the elementwise kernel
        return bwd_dact(gemm(dy, w_down.t().contiguous()), g, u, drop=drop, shard=shard, act=act)
    if inplace and not (g.is_contiguous() and u.is_contiguous()):
        raise ValueError("inplace=True needs contiguous g and u")
    dy, w_down, g, u = _c(dy), _c(w_down), _c(g), _c(u)
    M, K = dy.shape
    N = w_down.shape[1]
    d_gate = g if inplace else torch.empty((M, N), dtype=dt, device=dev)
    d_up = u if inplace else torch.empty((M, N), dtype=dt, device=dev)
    if M > 0:
        prob = _problem(M, K, N, dt, drop, shard, act, tuning)
        with _on(dev):
            check(load().gmlp_bwd_dhidden(C.byref(prob), ptr(dy), ptr(w_down), ptr(g), ptr(u),
                                          ptr(d_gate), ptr(d_up), stream_of(dy)))
    return d_gate, d_up


def bwd_dact(dh: Tensor, g: Tensor, u: Tensor, drop: Dropout = NO_DROPOUT, shard: Shard = NO_SHARD,
             act: str = "silu"):
    """(d_gate, d_up) from a caller-supplied dH."""
    dev = require_cuda(dh, g, u)
    dt = _same_dtype(dh, g, u)
    dh, g, u = _c(dh), _c(g), _c(u)
    M, N = dh.shape
    d_gate = torch.empty((M, N), dtype=dt, device=dev)
    d_up = torch.empty((M, N), dtype=dt, device=dev)
    if M > 0:
        prob = _problem(M, 8, N, dt, drop, shard, act)
        with _on(dev):
            check(load().gmlp_bwd_dact(C.byref(prob), ptr(dh), ptr(g), ptr(u), ptr(d_gate), ptr(d_up),
                                       stream_of(dh)))
    return d_gate, d_up


def bwd_dx(d_gate: Tensor, d_up: Tensor, w_gate: Tensor, w_up: Tensor, out: Tensor | None = None,
           tuning: int = 0) -> Tensor:
    """dx = d_gate W_gate + d_up W_up, written into `out` when given."""
    dev = require_cuda(d_gate, d_up, w_gate, w_up)
    dt = _same_dtype(d_gate, d_up, w_gate, w_up)
    if dt == torch.float32:
        # fp32 path: one K-major tf32 GEMM over the concatenated reduction [d_gate | d_up] . [W_gate ; W_up]
        dx32 = gemm(torch.cat((d_gate, d_up), dim=1), torch.cat((w_gate, w_up), dim=0).t().contiguous())
        if out is None:
            return dx32
        out.copy_(dx32)
        return out
    d_gate, d_up, w_gate, w_up = _c(d_gate), _c(d_up), _c(w_gate), _c(w_up)
    M, N = d_gate.shape
    K = w_gate.shape[1]
    dx = _out_buffer(out, (M, K), dt, dev)
    if M > 0:
        prob = _problem(M, K, N, dt, NO_DROPOUT, NO_SHARD, tuning=tuning)
        with _on(dev):
            check(load().gmlp_bwd_dx(C.byref(prob), ptr(d_gate), ptr(d_up), ptr(w_gate), ptr(w_up),
                                     ptr(dx), stream_of(d_gate)))
    return dx


_bias_scratch = {}


def bias_grad_scratch(K: int, N: int, dt: torch.dtype, dev: torch.device) -> Tensor:
    """Scratch of the fused bias-gradient sums (arrival counters, kept zero by the kernels, and fp32 partial
    sums) for a module of hidden size K and intermediate size N. One buffer per (device, stream, shape): calls
    on one stream are ordered, so they can share it. A new buffer is made when a kernel has given up a wait
    since (the counters may then be dirty)."""
    key = (dev, torch.cuda.current_stream(dev).cuda_stream, K, N, dt, _lib.scratch_epoch())
    buf = _bias_scratch.get(key)
    if buf is None:
        prob = _problem(8, K, N, dt, NO_DROPOUT, NO_SHARD)
        nbytes = load().gmlp_bias_grad_scratch_bytes(C.byref(prob))
        buf = torch.zeros(((nbytes + 3) // 4,), dtype=torch.int32, device=dev)
        if len(_bias_scratch) > 64:
            _bias_scratch.clear()
        _bias_scratch[key] = buf
    return buf


def bwd_dw_gate_up(d_gate: Tensor, d_up: Tensor, x: Tensor, tuning: int = 0, bias_grads: bool = False):
    """(dW_gate, dW_up) = (d_gate^T x, d_up^T x); with bias_grads=True also (db_gate, db_up), the column
    sums of d_gate and d_up, taken inside the same kernel."""
    dev = require_cuda(d_gate, d_up, x)
    dt = _same_dtype(d_gate, d_up, x)
    if dt == torch.float32 and d_gate.shape[0] > 0:
        # fp32 path: K-major tf32 GEMMs on transposed copies; bias gradients by the column-sum kernels
        xt = x.t().contiguous()
        dwg, dwu = gemm(d_gate.t().contiguous(), xt), gemm(d_up.t().contiguous(), xt)
        return (dwg, dwu, colsum(d_gate), colsum(d_up)) if bias_grads else (dwg, dwu)
    d_gate, d_up, x = _c(d_gate), _c(d_up), _c(x)
    M, N = d_gate.shape
    K = x.shape[1]
    if M == 0:
        z = lambda *s: torch.zeros(s, dtype=dt, device=dev)
        return (z(N, K), z(N, K), z(N), z(N)) if bias_grads else (z(N, K), z(N, K))
    dw_gate = torch.empty((N, K), dtype=dt, device=dev)
    dw_up = torch.empty((N, K), dtype=dt, device=dev)
    prob = _problem(M, K, N, dt, NO_DROPOUT, NO_SHARD, tuning=tuning)
    if not bias_grads:
        with _on(dev):
            check(load().gmlp_bwd_dw_gate_up(C.byref(prob), ptr(d_gate), ptr(d_up), ptr(x), ptr(dw_gate),
                                             ptr(dw_up), stream_of(x)))
        return dw_gate, dw_up
    db_gate = torch.empty((N,), dtype=dt, device=dev)
    db_up = torch.empty((N,), dtype=dt, device=dev)
    with _on(dev):
        scratch = bias_grad_scratch(K, N, dt, dev)
        check(load().gmlp_bwd_dw_gate_up_bias(C.byref(prob), ptr(d_gate), ptr(d_up), ptr(x), ptr(dw_gate), ptr(dw_up),
                                              ptr(db_gate), ptr(db_up), ptr(scratch),
                                              scratch.numel() * scratch.element_size(), stream_of(x)))
    return dw_gate, dw_up, db_gate, db_up


def bwd_dw_down(dy: Tensor, h: Tensor, tuning: int = 0, bias_grad: bool = False):
    """dW_down = dy^T h; with bias_grad=True returns (dW_down, db_down), db_down = column sums of dy from
    the same kernel."""
    dev = require_cuda(dy, h)
    dt = _same_dtype(dy, h)
    if dt == torch.float32 and dy.shape[0] > 0:
        dw32 = gemm(dy.t().contiguous(), h.t().contiguous())
        return (dw32, colsum(dy)) if bias_grad else dw32
    dy, h = _c(dy), _c(h)
    M, K = dy.shape
    N = h.shape[1]
    if M == 0:
        dw = torch.zeros((K, N), dtype=dt, device=dev)
        return (dw, torch.zeros((K,), dtype=dt, device=dev)) if bias_grad else dw
    dw = torch.empty((K, N), dtype=dt, device=dev)
    prob = _problem(M, K, N, dt, NO_DROPOUT, NO_SHARD, tuning=tuning)
    if not bias_grad:
        with _on(dev):
            check(load().gmlp_bwd_dw_down(C.byref(prob), ptr(dy), ptr(h), ptr(dw), stream_of(dy)))
        return dw
    db = torch.empty((K,), dtype=dt, device=dev)
    with _on(dev):
        scratch = bias_grad_scratch(K, N, dt, dev)
        check(load().gmlp_bwd_dw_down_bias(C.byref(prob), ptr(dy), ptr(h), ptr(dw), ptr(db), ptr(scratch),
                                           scratch.numel() * scratch.element_size(), stream_of(dy)))
    return dw, db


DECODE_MAX_TOKENS = 64


def decode_supported(M: int, K: int, N: int) -> bool:
    """Shapes the weight-streaming decode kernels accept."""
    return 0 < M <= DECODE_MAX_TOKENS and K % 64 == 0 and N % 64 == 0


def decode_scratch(M: int, K: int, N: int, dt: torch.dtype, device: torch.device) -> Tensor:
    """Zero-initialised scratch for decode_fwd (partial-tile slots + per-tile counters).

    Sized for up to 64 tokens, so one buffer serves every decode call of a module.
    The kernels leave the counters zero, so the buffer is reusable without clearing.
    """
    prob = _problem(DECODE_MAX_TOKENS, K, N, dt, NO_DROPOUT, NO_SHARD)
    with torch.cuda.device(device):
        nbytes = load().gmlp_decode_scratch_bytes(C.byref(prob))
    return torch.zeros(((nbytes + 3) // 4,), dtype=torch.int32, device=device)


def decode_fwd(x: Tensor, w_gate: Tensor, b_gate: Tensor | None, w_up: Tensor, b_up: Tensor | None,
               w_down: Tensor, b_down: Tensor | None, scratch: Tensor | None = None, act: str = "silu",
               residual: Tensor | None = None, out: Tensor | None = None, row_scale: Tensor | None = None,
               ordinary_launch: bool = False, one_launch: bool = False) -> Tensor:
    """y = (act(x W_gate^T + b_gate) * (x W_up^T + b_up)) W_down^T + b_down (+ residual) for M <= 64 tokens,
    written into `out` when given. one_launch=True runs both projections from one persistent kernel instead of
    two chained ones. The kernels normally start streaming weights while the preceding kernel
    on the stream is still running; ordinary_launch=True makes the call wait for it first (for the call that
    follows a kernel which writes the weights)."""
    dev = require_cuda(x, w_gate, b_gate, w_up, b_up, w_down, b_down, residual)
    dt = _same_dtype(x, w_gate, b_gate, w_up, b_up, w_down, b_down, residual)
    residual = _c(residual)
    x, w_gate, w_up, w_down = _c(x), _c(w_gate), _c(w_up), _c(w_down)
    b_gate, b_up, b_down = _c(b_gate), _c(b_up), _c(b_down)
    M, K = x.shape
    N = w_gate.shape[0]
    if not decode_supported(M, K, N):
        raise ValueError(f"decode path needs 1 <= M <= 64 and K, N multiples of 64; got M={M} K={K} N={N}")
    if scratch is None:
        scratch = decode_scratch(M, K, N, dt, dev)
    h = torch.empty((M, N), dtype=dt, device=dev)
    y = _out_buffer(out, (M, K), dt, dev)
    prob = _problem(M, K, N, dt, NO_DROPOUT, NO_SHARD, act, _lib.tune_word(ordinary_launch=ordinary_launch))
    _check_row_scale(row_scale, M, dev)
    with _on(dev):
        fn = load().gmlp_decode_fwd_fused if one_launch else load().gmlp_decode_fwd_scaled
        check(fn(C.byref(prob), ptr(x), ptr(row_scale), ptr(w_gate), ptr(b_gate), ptr(w_up),
                                            ptr(b_up), ptr(w_down), ptr(b_down), ptr(residual), ptr(h), ptr(y),
                                            ptr(scratch), scratch.numel() * scratch.element_size(), stream_of(x)))
    return y


E4M3_MAX = 448.0


def quantize_weight_rows_e4m3(w: Tensor):
    """One-off preparation of a weight matrix for the 8-bit decode path: (w8, scale) with w8 the e4m3
    bytes ([rows, cols] uint8) of w / scale[:, None] and scale[r] = amax|w[r, :]| / 448 (fp32), so that
    w ~= w8 * scale[:, None]. Plain torch ops: this runs when weights are loaded, not per step."""
    wf = w.detach().float()
    scale = (wf.abs().amax(dim=1).clamp_min(1e-30) / E4M3_MAX).contiguous()
    w8 = (wf / scale[:, None]).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
    return w8, scale


def quantize_rows_e4m3(x: Tensor):
    """Per-token dynamic quantisation on the GPU: (q, scale), q uint8 [M, K] holding e4m3(x / scale[:, None]),
    scale[m] = amax|x[m, :]| / 448 (fp32)."""
    dev = require_cuda(x)
    x = _c(x)
    M, K = x.shape
    q = torch.empty((M, K), dtype=torch.uint8, device=dev)
    scale = torch.empty((M,), dtype=torch.float32, device=dev)
    if M > 0:
        with _on(dev):
            check(load().gmlp_quantize_rows_e4m3(M, K, dtype_code(x.dtype), ptr(x), x.stride(0), ptr(q), ptr(scale),
                                                 stream_of(x)))
    return q, scale


def decode_fp8_supported(M: int, K: int, N: int) -> bool:
    return 0 < M <= DECODE_MAX_TOKENS and K % 128 == 0 and N % 128 == 0


def decode_fwd_fp8(x: Tensor, w_gate8: Tensor, w_gate_scale: Tensor, b_gate: Tensor | None, w_up8: Tensor,
                   w_up_scale: Tensor, b_up: Tensor | None, w_down8: Tensor, w_down_scale: Tensor,
                   b_down: Tensor | None, scratch: Tensor | None = None, act: str = "silu",
                   residual: Tensor | None = None, ordinary_launch: bool = False) -> Tensor:
    """decode_fwd on e4m3 weights (quantize_weight_rows_e4m3) with activations quantised per token on the fly;
    x, biases, residual and the result stay 16-bit."""
    dev = require_cuda(x, w_gate8, w_up8, w_down8, b_gate, b_up, b_down, residual)
    dt = _same_dtype(x, b_gate, b_up, b_down, residual)
    x, residual = _c(x), _c(residual)
    M, K = x.shape
    N = w_gate8.shape[0]
    for w8, sc, shape in ((w_gate8, w_gate_scale, (N, K)), (w_up8, w_up_scale, (N, K)), (w_down8, w_down_scale, (K, N))):
        if w8.dtype != torch.uint8 or tuple(w8.shape) != shape or not w8.is_contiguous():
            raise ValueError(f"8-bit weights must be contiguous uint8 of shape {shape}")
        if sc.dtype != torch.float32 or tuple(sc.shape) != (shape[0],) or not sc.is_contiguous():
            raise ValueError(f"weight scales must be contiguous float32 of shape ({shape[0]},)")
    if not decode_fp8_supported(M, K, N):
        raise ValueError(f"8-bit decode path needs 1 <= M <= 64 and K, N multiples of 128; got M={M} K={K} N={N}")
    if scratch is None:
        scratch = decode_scratch(M, K, N, dt, dev)
    x8 = torch.empty((M, K), dtype=torch.uint8, device=dev)
    xs = torch.empty((M,), dtype=torch.float32, device=dev)
    h = torch.empty((M, N), dtype=dt, device=dev)
    h8 = torch.empty((M, N), dtype=torch.uint8, device=dev)
    hs = torch.empty((M,), dtype=torch.float32, device=dev)
    y = torch.empty((M, K), dtype=dt, device=dev)
    prob = _problem(M, K, N, dt, NO_DROPOUT, NO_SHARD, act, _lib.tune_word(ordinary_launch=ordinary_launch))
    with _on(dev):
        check(load().gmlp_decode_fwd_fp8(C.byref(prob), ptr(x), ptr(w_gate8), ptr(w_gate_scale), ptr(b_gate), ptr(w_up8),
                                         ptr(w_up_scale), ptr(b_up), ptr(w_down8), ptr(w_down_scale), ptr(b_down),
                                         ptr(residual), ptr(x8), ptr(xs), ptr(h), ptr(h8), ptr(hs), ptr(y), ptr(scratch),
                                         scratch.numel() * scratch.element_size(), stream_of(x)))
    return y


def colsum(src: Tensor) -> Tensor:
    """Column sums of a [rows, cols] matrix (fp32 accumulation), in src's dtype."""
    dev = require_cuda(src)
    src = _c(src)
    rows, cols = src.shape
    if rows == 0:
        return torch.zeros((cols,), dtype=src.dtype, device=dev)
    lib = load()
    nbytes = lib.gmlp_colsum_scratch_bytes(rows, cols)
    scratch = torch.empty((nbytes // 4,), dtype=torch.float32, device=dev)
    dst = torch.empty((cols,), dtype=src.dtype, device=dev)
    with _on(dev):
        check(lib.gmlp_colsum(rows, cols, dtype_code(src.dtype), ptr(src), src.stride(0), ptr(scratch),
                              nbytes, ptr(dst), stream_of(src)))
    return dst


def dropout_mask(M: int, N: int, drop: Dropout, shard: Shard = NO_SHARD,
                 device: torch.device | str = "cuda") -> Tensor:
    """uint8 keep-mask [M, N] of the Philox dropout contract, generated on the GPU."""
    device = torch.device(device)
    mask = torch.empty((M, N), dtype=torch.uint8, device=device)
    prob = _problem(M, 8, N, torch.bfloat16, drop, shard)
    with torch.cuda.device(device):
        check(load().gmlp_dropout_mask(C.byref(prob), ptr(mask), torch.cuda.current_stream(device).cuda_stream))
    return mask


def gemm(a: Tensor, b: Tensor, a_mn: bool = False, b_mn: bool = False, bias: Tensor | None = None) -> Tensor:
    """C = A B^T on the tcgen05 engine. a_mn: `a` is stored [K, M]; b_mn: `b` is stored [K, N]."""
    dev = require_cuda(a, b, bias)
    dt = _same_dtype(a, b, bias)
    if dt == torch.float32 and (a_mn or b_mn):
        # the tf32 kernels take K-major operands only: transpose the MN-major ones once
        return gemm(a.t() if a_mn else a, b.t() if b_mn else b, bias=bias)
    a, b, bias = _c(a), _c(b), _c(bias)
    K, M = (a.shape if a_mn else a.shape[::-1])
    Kb, N = (b.shape if b_mn else b.shape[::-1])
    if K != Kb:
        raise ValueError(f"reduction extents differ: {K} vs {Kb}")
    c = torch.empty((M, N), dtype=dt, device=dev)
    with _on(dev):
        check(load().gmlp_gemm(dtype_code(dt), int(a_mn), int(b_mn), M, N, K, ptr(a), a.stride(0), ptr(b),
                               b.stride(0), ptr(c), c.stride(0), ptr(bias), stream_of(a)))
    return c
