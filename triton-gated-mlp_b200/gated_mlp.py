"""FusedGatedMLP: the reference's module API on sm_100a kernels.

Drop-in for the reference's FusedGatedMLP (src/triton_gated_mlp/gated_mlp.py:203-237):
same constructor keywords, parameter names (gate_proj / up_proj / down_proj, so
state_dicts and copy_weights keep working), attributes (hidden_size,
intermediate_size, act_fn, dropout) and forward(x) contract for any number of
leading dimensions. Semantics are those of EagerGatedMLP (:73-98): bias on all
three projections and dropout on the hidden state, which the reference's fused
path silently drops (:172-180, :200).

One autograd.Function spans all three projections. Forward: one tcgen05 kernel
for gate/up + bias + SiLU*up + dropout, one for the down projection. Backward:
dH fused with the activation derivative, then dX, dW_gate/dW_up and dW_down with
the bias gradients (column sums of d_gate, d_up, dy) taken inside the weight-gradient
kernels; the gate / up pre-activations are saved, not recomputed.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor, nn
from torch.autograd.function import Function

from .ops import kernels
from .ops.fwd import SUPPORTED_ACTS, mlp_hidden_states_fwd  # noqa: F401  (re-exported like the reference)
from .ops.bwd import mlp_hidden_states_bwd  # noqa: F401
from .ops.kernels import Dropout, Shard
from . import _lib, parallel


# torch twins of the gate activations, kept as `module.act` like the reference does (gated_mlp.py:218).
_ACT_MODULES = {
    "silu": nn.SiLU, "swish": nn.SiLU, "no_act": nn.Identity, "relu": nn.ReLU, "gelu": nn.GELU,
    "sigmoid": nn.Sigmoid, "tanh": nn.Tanh, "leaky_relu": nn.LeakyReLU,
}


class _SmLimit:
    """While switched on, GEMM launches that pass `limit.tuning` leave `comm_sms` SMs free of
    persistent CTAs for a collective's kernels. The limit travels with each call
    (gmlp_problem_t.tuning); nothing process-wide is touched, so other modules, devices and
    host threads keep their full grids."""

    def __init__(self, device: torch.device, comm_sms: int, sm_count: Optional[int] = None):
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(device).multi_processor_count
        self.sms = max(2, int(sm_count) - max(0, int(comm_sms)))
        self.on = False

    def __call__(self, on: bool) -> None:
        self.on = bool(on)

    @property
    def tuning(self) -> int:
        return _lib.tune_word(sm_limit=self.sms) if self.on else 0


class FusedGatedMLPFunction(Function):
    """y = down(dropout(silu(gate(x)) * up(x))) with hand-written forward and backward.

    Replaces the reference's FusedGatedMLPFunction (gated_mlp.py:159-200), which
    covers only the gate/up half and returns no bias gradients.
    """

    @staticmethod
    def forward(ctx, x: Tensor, W_gate: Tensor, b_gate: Optional[Tensor], W_up: Tensor,
                b_up: Optional[Tensor], W_down: Tensor, b_down: Optional[Tensor],
                drop: Dropout, shard: Shard, tp_group, act: str = "silu",
                residual: Optional[Tensor] = None, tp_chunk_rows=(0, 0), tp_comm_sms: int = 16,
                inplace_backward: bool = True, peer_sum=None) -> Tensor:
        tp_chunk_fwd, tp_chunk_bwd = tp_chunk_rows
        need_bwd = any(ctx.needs_input_grad)
        # With the intermediate dimension sharded, every rank holds a partial sum
        # of y; the output bias is added once, by the rank that owns column 0.
        owner = tp_group is None or shard.col0 == 0
        bias, res = (b_down if owner else None), (residual if owner else None)
        if tp_group is not None and tp_chunk_fwd > 0:
            if need_bwd:
                h, g, u = kernels.hidden_fwd(x, W_gate, b_gate, W_up, b_up, drop=drop, shard=shard, save=True, act=act)
            else:
                h = kernels.hidden_fwd(x, W_gate, b_gate, W_up, b_up, drop=drop, shard=shard, save=False, act=act)
                g = u = None
            # Down projection chunk by chunk over the token rows: chunk i's all-reduce
            # (NCCL, on its own stream) runs beside chunk i+1's GEMM.
            y = torch.empty((x.shape[0], W_down.shape[0]), dtype=x.dtype, device=x.device)
            limit = _SmLimit(x.device, tp_comm_sms)
            works = parallel.overlapped_all_reduce(
                y, lambda r0, r1: kernels.down_fwd(h[r0:r1], W_down, bias, None if res is None else res[r0:r1],
                                                   out=y[r0:r1], tuning=limit.tuning),
                tp_group, tp_chunk_fwd, limit)
            parallel.wait_all(works)
        elif (tp_group is not None and peer_sum is not None
              and peer_sum.supports_down_sum(x.shape[0], W_down.shape[0], x.dtype)):
            # the down projection scatters its partial output into the owners' inboxes from its epilogue;
            # one more kernel per rank sums and hands round (no NCCL call on this path)
            if need_bwd:
                h, g, u = kernels.hidden_fwd(x, W_gate, b_gate, W_up, b_up, drop=drop, shard=shard, save=True, act=act)
            else:
                h = kernels.hidden_fwd(x, W_gate, b_gate, W_up, b_up, drop=drop, shard=shard, save=False, act=act)
                g = u = None
            y = peer_sum.down_fwd_sum(h, W_down, bias, res)
        else:
            # both kernels from one library call
            y, h, g, u = kernels.mlp_fwd(x, W_gate, b_gate, W_up, b_up, W_down, bias, drop=drop, shard=shard,
                                         save=need_bwd, act=act, residual=res)
            if tp_group is not None:
                parallel.all_reduce_sum(y, tp_group)
        if need_bwd:
            ctx.save_for_backward(x, W_gate, W_up, W_down, g, u, h)
            ctx.drop, ctx.shard, ctx.tp_group, ctx.act = drop, shard, tp_group, act
            ctx.tp_chunk_rows, ctx.tp_comm_sms = tp_chunk_bwd, tp_comm_sms
            ctx.has_bias = (b_gate is not None, b_up is not None, b_down is not None)
            ctx.inplace_backward, ctx.consumed = bool(inplace_backward), False
            ctx.peer_sum = peer_sum if tp_group is not None else None
        return y

    @staticmethod
    def backward(ctx, dy: Tensor):
        x, W_gate, W_up, W_down, g, u, h = ctx.saved_tensors
        need = ctx.needs_input_grad
        dy = dy.contiguous()
        dx = dW_gate = db_gate = dW_up = db_up = dW_down = db_down = None
        need_hidden = need[0] or need[1] or need[2] or need[3] or need[4]
        if need_hidden:
            if ctx.consumed:
                raise RuntimeError(
                    "FusedGatedMLP: this graph's saved gate/up pre-activations were overwritten by an earlier "
                    "backward pass (inplace_backward=True writes d_gate / d_up over them). Set "
                    "module.inplace_backward = False to run backward more than once over one forward.")
            if dy.dtype == torch.float32:
                ctx.inplace_backward = False   # the fp32 path composes the pass from separate kernels
            ctx.consumed = ctx.inplace_backward
        # The bias gradients are column sums of d_gate / d_up / dy; the weight-gradient GEMMs deliver
        # them on the side (their A operand is exactly that matrix, transposed). Only a caller that
        # wants a bias gradient without its weight gradient pays a separate pass.
        want_bg, want_bu, want_bd = need[2] and ctx.has_bias[0], need[4] and ctx.has_bias[1], need[6] and ctx.has_bias[2]
        want_wgu = need[1] or need[3]
        works = []
        # (an explicit tp_chunk_rows keeps the chunked NCCL overlap, which is the faster of the two at eight ranks)
        use_push = (ctx.tp_group is not None and ctx.peer_sum is not None and need[0] and dy.dtype != torch.float32
                    and ctx.tp_chunk_rows == 0
                    and ctx.peer_sum.supports_down_sum(x.shape[0], x.shape[1], x.dtype))
        if use_push:
            # dx scattered into the owners' inboxes from its GEMM's epilogue; the sum kernel goes behind the
            # weight-gradient GEMMs (no NCCL call in the pass)
            d_gate, d_up = kernels.bwd_dhidden(dy, W_down, g, u, drop=ctx.drop, shard=ctx.shard, act=ctx.act,
                                               inplace=ctx.inplace_backward)
            dx = ctx.peer_sum.dx_push(d_gate, d_up, W_gate, W_up)
            if want_wgu:
                if want_bg or want_bu:
                    dW_gate, dW_up, db_gate, db_up = kernels.bwd_dw_gate_up(d_gate, d_up, x, bias_grads=True)
                else:
                    dW_gate, dW_up = kernels.bwd_dw_gate_up(d_gate, d_up, x)
            if need[5]:
                if want_bd:
                    dW_down, db_down = kernels.bwd_dw_down(dy, h, bias_grad=True)
                else:
                    dW_down = kernels.bwd_dw_down(dy, h)
            ctx.peer_sum.finish_sum(dx)
        elif ctx.tp_group is not None and ctx.tp_chunk_rows > 0 and need[0]:
            # dx chunk by chunk; the last chunk's all-reduce runs beside the weight-gradient GEMMs
            limit = _SmLimit(x.device, ctx.tp_comm_sms)
            d_gate, d_up = kernels.bwd_dhidden(dy, W_down, g, u, drop=ctx.drop, shard=ctx.shard, act=ctx.act,
                                               inplace=ctx.inplace_backward)
            dx = torch.empty((x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
            works = parallel.overlapped_all_reduce(
                dx, lambda r0, r1: kernels.bwd_dx(d_gate[r0:r1], d_up[r0:r1], W_gate, W_up, out=dx[r0:r1],
                                                  tuning=limit.tuning),
                ctx.tp_group, ctx.tp_chunk_rows, limit)
            limit(True)
            if want_wgu:
                if want_bg or want_bu:
                    dW_gate, dW_up, db_gate, db_up = kernels.bwd_dw_gate_up(d_gate, d_up, x, tuning=limit.tuning,
                                                                            bias_grads=True)
                else:
                    dW_gate, dW_up = kernels.bwd_dw_gate_up(d_gate, d_up, x, tuning=limit.tuning)
            if need[5]:
                if want_bd:
                    dW_down, db_down = kernels.bwd_dw_down(dy, h, tuning=limit.tuning, bias_grad=True)
                else:
                    dW_down = kernels.bwd_dw_down(dy, h, tuning=limit.tuning)
        else:
            # every kernel of the pass from one library call
            r = kernels.mlp_bwd(dy, x, W_gate, W_up, W_down, g, u, h, drop=ctx.drop, shard=ctx.shard, act=ctx.act,
                                want_dx=bool(need[0]), want_dw_gate_up=bool(want_wgu), want_dw_down=bool(need[5]),
                                want_db_gate=bool(want_bg and want_wgu), want_db_up=bool(want_bu and want_wgu),
                                want_db_down=bool(want_bd and need[5]), inplace=ctx.inplace_backward) \
                if (need_hidden or need[5]) else {}
            dx, dW_gate, dW_up, dW_down = r.get("dx"), r.get("dw_gate"), r.get("dw_up"), r.get("dw_down")
            db_gate, db_up, db_down = r.get("db_gate"), r.get("db_up"), r.get("db_down")
            d_gate, d_up = r.get("d_gate"), r.get("d_up")
            if dx is not None and ctx.tp_group is not None:
                parallel.all_reduce_sum(dx, ctx.tp_group)
        # bias gradients asked for without their weight gradients: stand-alone column sums
        if (want_bg or want_bu) and not want_wgu:
            if d_gate is None:
                d_gate, d_up = kernels.bwd_dhidden(dy, W_down, g, u, drop=ctx.drop, shard=ctx.shard, act=ctx.act,
                                                   inplace=ctx.inplace_backward)
            db_gate = kernels.colsum(d_gate) if want_bg else None
            db_up = kernels.colsum(d_up) if want_bu else None
        if not want_bg:
            db_gate = None
        if not want_bu:
            db_up = None
        if want_bd and not need[5]:
            db_down = kernels.colsum(dy)
        parallel.wait_all(works)
        d_res = dy if (len(need) > 11 and need[11]) else None  # y = ... + residual
        return (dx, dW_gate, db_gate, dW_up, db_up, dW_down, db_down, None, None, None, None, d_res, None, None,
                None, None)


class _InputRMSNorm(Function):
    """x / rms(x) * weight for the training path (the inference path never writes the normalised
    activations: see FusedGatedMLP.attach_input_norm). Row statistics and both passes over the rows are
    library kernels; the products with `weight` are elementwise torch ops on [M, K]."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, eps: float) -> Tensor:
        rs, xn = kernels.rms_rowscale(x, eps, normalised=True)
        ctx.save_for_backward(xn, rs, weight)
        return xn * weight

    @staticmethod
    def backward(ctx, dout: Tensor):
        xn, rs, weight = ctx.saved_tensors
        dout = dout.contiguous()
        dw = (dout.float() * xn.float()).sum(0).to(weight.dtype) if ctx.needs_input_grad[1] else None
        dx = kernels.rms_bwd(dout * weight, xn, rs) if ctx.needs_input_grad[0] else None
        return dx, dw, None


class FusedGatedMLP(nn.Module):
    """Gated MLP block; see the module docstring.

    The tuned kernels compute in bfloat16 or float16 with fp32 accumulation: cast the
    module with .to(torch.bfloat16) or .to(torch.float16) (and move it to a CUDA device).
    A module left in float32, as the reference's own tests build it, runs too: its products
    are taken in tf32 (tcgen05.mma.kind::tf32, 10-bit mantissa, fp32 accumulation; the
    tolerance class of the reference's GPU tests, atol 1e-3) through the K-major kernels,
    with transposed copies where the backward pass needs them: a compatibility path, not
    a fast one (no decode kernels, no input norm, no 8-bit weights). A CPU tensor raises
    GmlpError.

    Extra keyword-only arguments (all default to the single-GPU reference behaviour):
      parallel_mode  "none" | "token" | "tp". "token": this rank holds a slice of
                     the token rows and full weights; no communication, only the
                     dropout mask is offset by `token_row0`. "tp": this rank's
                     parameters are the rank-th slice of the intermediate
                     dimension (intermediate_size is the LOCAL size) and the
                     down-projection partial sums are all-reduced over
                     `process_group`.
      process_group  torch.distributed group for "tp".
    Attributes (set after construction):
      inplace_backward  True (default): the backward pass writes d_gate / d_up over the saved
                     gate / up pre-activations instead of allocating two more [M, N]
                     buffers. A second backward over the same forward (retain_graph=True)
                     then raises; set False for that use.
      tp_chunk_rows  "tp" at prefill / training sizes. 0 (default): one all-reduce after
                     the whole dx GEMM of the backward pass. > 0: that GEMM runs in chunks
                     of this many token rows and each chunk's all-reduce overlaps the next
                     chunk's GEMM, the last one the weight-gradient GEMMs.
      tp_chunk_rows_fwd  the same for the down projection of the forward pass, where
                     nothing follows the last chunk to hide its all-reduce behind (off by
                     default).
      tp_comm_sms    SMs the persistent GEMM grids leave to the collective's kernels
                     while one is in flight (default 16).
      peer_max_bytes largest partial output the "tp" decode path sums through peer memory
                     (after enable_peer_allreduce()); larger ones go through NCCL.
      check_status_every  0 (default): never read the device status word on the decode
                     path. N > 0: every N-th "tp" decode call synchronises, reads it and
                     raises if a peer wait ran out (the output of that call is then this
                     rank's partial sum only).
      philox_seed    dropout seed; `philox_offset` advances by one per training
                     forward call.
    """

    def __init__(
        self,
        hidden_size: int = 256,
        intermediate_size: int = 512,
        bias: bool = True,
        hidden_act: str = "silu",
        dropout_p: float = 0.0,
        *,
        parallel_mode: str = "none",
        process_group=None,
        tp_rank: Optional[int] = None,
        tp_size: Optional[int] = None,
        philox_seed: int = 0,
    ):
        super().__init__()
        if hidden_act not in SUPPORTED_ACTS:
            raise NotImplementedError(f"gate activation {hidden_act!r}: supported are {sorted(SUPPORTED_ACTS)}")
        if parallel_mode not in ("none", "token", "tp"):
            raise ValueError(f"parallel_mode {parallel_mode!r} not in ('none', 'token', 'tp')")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.gate_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=bias)
        self.up_proj = nn.Linear(self.hidden_size, self.intermediate_size, bias=bias)
        self.down_proj = nn.Linear(self.intermediate_size, self.hidden_size, bias=bias)
        self.act = _ACT_MODULES[hidden_act]()
        self.act_fn = hidden_act
        self.dropout = nn.Dropout(dropout_p)
        self.parallel_mode = parallel_mode
        self.process_group = process_group
        if parallel_mode == "tp":
            self.tp_rank, self.tp_size = parallel.resolve_rank_size(process_group, tp_rank, tp_size)
        else:
            self.tp_rank, self.tp_size = 0, 1
        self.token_row0 = 0
        self.philox_seed = int(philox_seed)
        self.philox_offset = 0
        self._decode_scratch = None
        self._peer = None
        self._peer_sum = None
        self.inplace_backward = True
        self.tp_chunk_rows = 0
        self.tp_chunk_rows_fwd = 0
        self.tp_comm_sms = 16
        self.peer_max_bytes = 1024 * 1024
        self.check_status_every = 0
        self.decode_one_launch = False   # both decode projections from one persistent kernel (16-bit weights)
        self._decode_calls = 0
        self.input_norm_weight = None
        self.input_norm_eps = 1e-6
        self._folded = None
        self._fp8 = None
        self._decode_weight_versions = None

    def attach_input_norm(self, weight: Tensor, eps: float = 1e-6) -> None:
        """Put an RMSNorm in front of the MLP: forward(x) becomes MLP(x / rms(x) * weight), the step that
        precedes the MLP in a Llama block (no counterpart in the reference, whose module starts at the
        projections, gated_mlp.py:224-227). `weight` ([hidden_size]) becomes the parameter
        `input_norm_weight`. Without gradients the norm costs one pass over x for the row statistics: the
        weight is folded into copies of W_gate / W_up (refreshed whenever a parameter changes) and 1 / rms is
        applied to the accumulators of the gate/up kernel, so the normalised activations are never written.
        With gradients the normalised activations are materialised once and the norm's backward is a
        row-wise kernel of its own."""
        if weight.shape != (self.hidden_size,):
            raise ValueError(f"norm weight must have shape ({self.hidden_size},), got {tuple(weight.shape)}")
        self.input_norm_weight = nn.Parameter(weight.detach().clone().to(self.gate_proj.weight.device,
                                                                          self.gate_proj.weight.dtype))
        self.input_norm_eps = float(eps)
        self._folded = None

    def quantize_decode_weights(self, enable: bool = True) -> None:
        """Prepare (or drop) e4m3 copies of the three weight matrices, one scale per weight row, for the
        decode path: inference with at most 64 tokens then streams half the weight bytes (activations
        are quantised per token on the fly; everything else stays 16-bit). Call again after the weights
        change. Needs hidden and intermediate sizes that are multiples of 128; not combined with an
        attached input norm or tensor parallelism."""
        if not enable:
            self._fp8 = None
            return
        if self.input_norm_weight is not None or self.parallel_mode == "tp":
            raise NotImplementedError("8-bit decode weights are not combined with an input norm or tensor parallelism")
        if self.hidden_size % 128 or self.intermediate_size % 128:
            raise ValueError("8-bit decode weights need hidden_size and intermediate_size multiples of 128")
        q = kernels.quantize_weight_rows_e4m3
        self._fp8 = (q(self.gate_proj.weight), q(self.up_proj.weight), q(self.down_proj.weight))
        self._decode_weight_versions = None     # the next decode call follows the kernels that wrote the copies

    def _folded_weights(self):
        """(W_gate * weight, W_up * weight), cached until any of the three tensors is modified."""
        key = (self.gate_proj.weight._version, self.up_proj.weight._version, self.input_norm_weight._version,
               self.gate_proj.weight.data_ptr(), self.up_proj.weight.data_ptr(), self.input_norm_weight.data_ptr())
        if self._folded is None or self._folded[0] != key:
            with torch.no_grad():
                w = self.input_norm_weight
                self._folded = (key, (self.gate_proj.weight * w).contiguous(), (self.up_proj.weight * w).contiguous())
        return self._folded[1], self._folded[2]

    def set_philox(self, seed: int, offset: int = 0) -> None:
        self.philox_seed, self.philox_offset = int(seed), int(offset)

    def _shard(self) -> Shard:
        if self.parallel_mode == "tp":
            return Shard(row0=0, col0=self.tp_rank * self.intermediate_size,
                         n_global=self.tp_size * self.intermediate_size)
        if self.parallel_mode == "token":
            return Shard(row0=int(self.token_row0), col0=0, n_global=self.intermediate_size)
        return Shard()

    def _decode_forward(self, x: Tensor, tp_group, residual: Optional[Tensor]) -> Tensor:
        """Inference with at most 64 tokens: the weight-streaming kernels (HBM-bound)."""
        # A kernel that gave up a wait may have left counters in the scratch non-zero: a
        # non-zero status read (anywhere in the process) starts a new scratch epoch.
        key = (x.device, x.dtype, _lib.scratch_epoch())
        if self._decode_scratch is None or self._decode_scratch[0] != key:
            self._decode_scratch = (key, kernels.decode_scratch(
                x.shape[0], self.hidden_size, self.intermediate_size, x.dtype, x.device))
        # The decode kernels begin to stream weights while the kernel ahead of them on the stream is still
        # running. If a parameter has been modified in place since the last decode call (an optimiser step, a
        # weight merge), that kernel may be the writer: this one call starts as an ordinary launch.
        versions = (self.gate_proj.weight._version, self.up_proj.weight._version, self.down_proj.weight._version)
        ordinary = versions != self._decode_weight_versions
        self._decode_weight_versions = versions
        if self._fp8 is not None and tp_group is None:
            (wg8, wgs), (wu8, wus), (wd8, wds) = self._fp8
            return kernels.decode_fwd_fp8(x, wg8, wgs, self.gate_proj.bias, wu8, wus, self.up_proj.bias, wd8, wds,
                                          self.down_proj.bias, scratch=self._decode_scratch[1], act=self.act_fn,
                                          residual=residual, ordinary_launch=ordinary)
        own_bias = tp_group is None or self.tp_rank == 0
        w_gate, w_up, rs = self.gate_proj.weight, self.up_proj.weight, None
        if self.input_norm_weight is not None:
            (w_gate, w_up), rs = self._folded_weights(), kernels.rms_rowscale(x, self.input_norm_eps)
        y = kernels.decode_fwd(x, w_gate, self.gate_proj.bias, w_up,
                               self.up_proj.bias, self.down_proj.weight,
                               self.down_proj.bias if own_bias else None, scratch=self._decode_scratch[1],
                               act=self.act_fn, residual=residual if own_bias else None, row_scale=rs,
                               ordinary_launch=ordinary, one_launch=self.decode_one_launch)
        if tp_group is not None:
            if (self._peer is not None and self._peer.supports(y)
                    and y.numel() * y.element_size() <= self.peer_max_bytes):
                # The partial outputs are summed through the peers' memory, in place, as an
                # ordinary launch (as a programmatic dependent its blocks would occupy SMs that
                # the down projection's last CTAs still need).
                self._peer.all_reduce(y, out=y, dependent=False)
                self._decode_calls += 1
                if self.check_status_every > 0 and self._decode_calls % self.check_status_every == 0:
                    code = _lib.status_read(x.device)
                    if code != 0:
                        raise _lib.GmlpError(
                            f"device status {code}: a bounded wait ran out during tensor-parallel decode "
                            "(4 = a peer's partial output never arrived); the last output is not the full sum")
            else:
                parallel.all_reduce_sum(y, tp_group)
        return y

    def enable_peer_allreduce(self, max_tokens: int = 64) -> "parallel.PeerAllReduce":
        """Collective over the tensor-parallel group: from now on the decode path sums its partial
        outputs with the one-shot peer-memory kernel instead of an NCCL all-reduce. Call after the
        module has been moved to its device and dtype."""
        if self.parallel_mode != "tp":
            raise ValueError("enable_peer_allreduce applies to parallel_mode='tp'")
        group = self.process_group if self.process_group is not None else parallel.default_group()
        w = self.down_proj.weight
        self._peer = parallel.PeerAllReduce(group, int(max_tokens) * self.hidden_size, w.dtype, w.device)
        return self._peer

    def enable_peer_output_sum(self, max_tokens: int) -> "parallel.PeerAllReduce":
        """Collective over the tensor-parallel group: from now on the prefill / training forward of up to
        `max_tokens` rows (a multiple of 32 * world per call) sums its partial outputs without NCCL: the down
        projection pushes the other ranks' row blocks into their inboxes from its epilogue while it computes,
        and one more kernel adds and hands round (PeerAllReduce.down_fwd_sum). Each rank sets aside
        2 * world * max_tokens * hidden_size * 2 bytes for the inboxes. The backward pass keeps NCCL for dx."""
        if self.parallel_mode != "tp":
            raise ValueError("enable_peer_output_sum applies to parallel_mode='tp'")
        group = self.process_group if self.process_group is not None else parallel.default_group()
        w = self.down_proj.weight
        self._peer_sum = parallel.PeerAllReduce(group, int(max_tokens) * self.hidden_size, w.dtype, w.device)
        return self._peer_sum

    def forward(self, x: Tensor, residual: Optional[Tensor] = None) -> Tensor:
        """y = down(dropout(act(gate(x)) * up(x))) (+ residual, fused into the down projection's epilogue;
        the reference adds a residual outside the module, after gated_mlp.py:236-237)."""
        shapes = x.shape
        if len(shapes) > 2:
            x = x.reshape(-1, shapes[-1])
        if residual is not None:
            if residual.shape != shapes:
                raise ValueError(f"residual shape {tuple(residual.shape)} != input shape {tuple(shapes)}")
            residual = residual.reshape(-1, shapes[-1])
        p = float(self.dropout.p) if self.training else 0.0
        drop = Dropout(p, self.philox_seed, self.philox_offset)
        if p > 0.0:
            self.philox_offset += 1
        tp_group = self.process_group if self.parallel_mode == "tp" else None
        if self.parallel_mode == "tp" and tp_group is None:
            tp_group = parallel.default_group()
        needs_grad = torch.is_grad_enabled() and (
            x.requires_grad or any(q.requires_grad for q in self.parameters())
            or (residual is not None and residual.requires_grad))
        if x.dtype == torch.float32 and self.input_norm_weight is not None:
            raise NotImplementedError("the input norm is not available for float32 modules")
        if (not needs_grad and p == 0.0 and x.is_cuda and x.dtype != torch.float32
                and kernels.decode_supported(x.shape[0], self.hidden_size, self.intermediate_size)):
            y = self._decode_forward(x, tp_group, residual)
            return y.view(shapes) if len(shapes) > 2 else y
        if self.input_norm_weight is not None:
            if not needs_grad:
                # 1 / rms on the gate/up accumulators, norm weight folded into the weights
                w_gate, w_up = self._folded_weights()
                h = kernels.hidden_fwd(x, w_gate, self.gate_proj.bias, w_up, self.up_proj.bias, drop=drop,
                                       shard=self._shard(), act=self.act_fn,
                                       row_scale=kernels.rms_rowscale(x, self.input_norm_eps))
                own = tp_group is None or self.tp_rank == 0
                y = kernels.down_fwd(h, self.down_proj.weight, self.down_proj.bias if own else None,
                                     residual if own else None)
                if tp_group is not None:
                    parallel.all_reduce_sum(y, tp_group)
                return y.view(shapes) if len(shapes) > 2 else y
            x = _InputRMSNorm.apply(x, self.input_norm_weight, self.input_norm_eps)
        y = FusedGatedMLPFunction.apply(
            x, self.gate_proj.weight, self.gate_proj.bias, self.up_proj.weight, self.up_proj.bias,
            self.down_proj.weight, self.down_proj.bias, drop, self._shard(), tp_group, self.act_fn, residual,
            (int(self.tp_chunk_rows_fwd), int(self.tp_chunk_rows)) if tp_group is not None else (0, 0),
            int(self.tp_comm_sms), bool(self.inplace_backward), self._peer_sum if tp_group is not None else None,
        )
        return y.view(shapes) if len(shapes) > 2 else y
