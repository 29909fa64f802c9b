"""Host-side sharding logic for the two multi-GPU modes (one process per GPU).

token mode  Rows of x / y / dy / dx are split across ranks, weights are
            replicated, and no collective runs on the data path. Weight
            gradients are rank-local partial sums.
tp mode     The intermediate dimension is split: rank r owns rows
            [r*N/g, (r+1)*N/g) of W_gate / W_up (and of their biases) and the
            same columns of W_down. Forward all-reduces the partial y, backward
            all-reduces the partial dx; both over NCCL (NVLink / NVSwitch).

The reference has no multi-GPU code; this module is new. Everything here is plain
index arithmetic plus torch.distributed calls, so it is tested on CPU ranks with
the gloo backend.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def token_shard_range(m_global: int, rank: int, world: int) -> Tuple[int, int]:
    """(first row, row count) of `rank`'s contiguous slice; earlier ranks take the remainder."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(m_global, world)
    rows = base + (1 if rank < rem else 0)
    row0 = rank * base + min(rank, rem)
    return row0, rows


def tp_shard_range(n_global: int, rank: int, world: int, multiple: int = 16) -> Tuple[int, int]:
    """(first column, column count) of `rank`'s slice of the intermediate dimension.

    Every slice must be a multiple of `multiple` columns (the kernels need N % 16 == 0
    and the dropout index space needs column offsets that are multiples of 4).
    """
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_global % (world * multiple) != 0:
        raise ValueError(
            f"intermediate size {n_global} is not divisible into {world} shards of a multiple of {multiple}"
        )
    cols = n_global // world
    return rank * cols, cols


def shard_tp_state_dict(full: Dict[str, Tensor], rank: int, world: int) -> Dict[str, Tensor]:
    """Slice a full gate_proj/up_proj/down_proj state_dict down to `rank`'s tensor-parallel shard."""
    n_global = full["gate_proj.weight"].shape[0]
    c0, cols = tp_shard_range(n_global, rank, world)
    out = {}
    for name, t in full.items():
        if name in ("gate_proj.weight", "up_proj.weight", "gate_proj.bias", "up_proj.bias"):
            out[name] = t[c0:c0 + cols].clone()
        elif name == "down_proj.weight":
            out[name] = t[:, c0:c0 + cols].clone()
        else:  # down_proj.bias is replicated
            out[name] = t.clone()
    return out


def gather_tp_grads(local: Dict[str, Tensor], group=None) -> Dict[str, Tensor]:
    """All-gather sharded parameter gradients back into full-size tensors (for checks, not the hot path)."""
    world = dist.get_world_size(group)
    out = {}
    for name, t in local.items():
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=group)
        if name == "down_proj.weight":
            out[name] = torch.cat(parts, dim=1)
        elif name == "down_proj.bias":
            out[name] = parts[0]
        else:
            out[name] = torch.cat(parts, dim=0)
    return out


def default_group():
    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError("parallel_mode='tp' needs an initialised torch.distributed process group")
    return dist.group.WORLD


def resolve_rank_size(group, rank: Optional[int], size: Optional[int]) -> Tuple[int, int]:
    if rank is not None and size is not None:
        return int(rank), int(size)
    g = group if group is not None else default_group()
    return dist.get_rank(g), dist.get_world_size(g)


def all_reduce_sum(t: Tensor, group) -> Tensor:
    """In-place sum over the tensor-parallel group on the tensor's current stream."""
    if dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def chunk_ranges(m: int, rows: int) -> List[Tuple[int, int]]:
    """Row ranges [r0, r1) of at most `rows` rows covering [0, m); one range when rows <= 0 or rows >= m."""
    if m <= 0:
        return []
    if rows <= 0 or rows >= m:
        return [(0, m)]
    return [(r0, min(m, r0 + rows)) for r0 in range(0, m, rows)]


def overlapped_all_reduce(out: Tensor, produce: Callable[[int, int], None], group, chunk_rows: int,
                          limit_sms: Optional[Callable[[bool], None]] = None) -> list:
    """Fill `out` chunk by chunk and sum every chunk over `group` while the next one is being computed.

    `produce(r0, r1)` enqueues the kernels that write this rank's partial rows out[r0:r1] on the
    current stream. Each chunk's all-reduce is started asynchronously right behind its kernels (NCCL
    runs it on its own stream, ordered after them), so it runs beside the next chunk's kernels.
    `limit_sms(True)` is called before the first launch that shares the GPU with a collective and
    `limit_sms(False)` is left to the caller, who may want later kernels to keep sharing: persistent
    GEMM grids otherwise hold every SM and the collective's CTAs could not start before the GEMM ends.
    Returns the outstanding work handles; the caller waits on them (`wait_all`) before `out` is read.
    """
    works = []
    if dist.get_world_size(group) == 1:
        produce(0, out.shape[0])
        return works
    for i, (r0, r1) in enumerate(chunk_ranges(out.shape[0], chunk_rows)):
        if i == 1 and limit_sms is not None:
            limit_sms(True)
        produce(r0, r1)
        works.append(dist.all_reduce(out[r0:r1], op=dist.ReduceOp.SUM, group=group, async_op=True))
    return works


def wait_all(works: list) -> None:
    """Make the current stream (or, on CPU ranks, the host) wait for the collectives in `works`."""
    for w in works:
        w.wait()


class _LibPeerBackend:
    """The libgmlp side of PeerAllReduce: CUDA IPC regions and the one-shot reduction kernel."""

    def __init__(self, device: torch.device):
        import ctypes as C

        from . import _lib
        self._C, self._lib_mod, self.device = C, _lib, device
        self.lib = _lib.load()

    def region_bytes(self, max_elems: int, world: int) -> int:
        return int(self.lib.gmlp_peer_region_bytes(max_elems, world))

    def alloc(self, nbytes: int):
        C = self._C
        p, handle = C.c_void_p(), C.create_string_buffer(64)
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_peer_alloc(nbytes, C.byref(p), handle))
        return int(p.value), bytes(handle.raw)

    def open(self, handle: bytes) -> int:
        C = self._C
        p = C.c_void_p()
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_peer_open(handle, C.byref(p)))
        return int(p.value)

    def close(self, ptr: int) -> None:
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_peer_close(ptr))

    def free(self, ptr: int) -> None:
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_peer_free(ptr))

    def allreduce(self, dtype: torch.dtype, n: int, max_elems: int, src: Tensor, regions, rank: int, world: int,
                  dst: Tensor, dependent: bool) -> None:
        C = self._C
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_peer_allreduce(
                self._lib_mod.dtype_code(dtype), n, max_elems, src.data_ptr(), (C.c_void_p * world)(*regions),
                rank, world, dst.data_ptr(), 1 if dependent else 0,
                torch.cuda.current_stream(self.device).cuda_stream))


    def down_push_sum(self, prob, h: Tensor, w_down: Tensor, b_down, residual, y: Tensor, max_elems: int, regions,
                      rank: int, world: int) -> None:
        """gmlp_down_fwd_push followed by gmlp_peer_reduce_gather on the current stream."""
        C = self._C
        ptr = lambda t: None if t is None else t.data_ptr()
        st = torch.cuda.current_stream(self.device).cuda_stream
        regs = (C.c_void_p * world)(*regions)
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_down_fwd_push(
                C.byref(prob), ptr(h), ptr(w_down), ptr(b_down), ptr(residual), ptr(y), max_elems, regs, rank, world,
                st))
            self._lib_mod.check(self.lib.gmlp_peer_reduce_gather(
                self._lib_mod.dtype_code(y.dtype), y.numel(), max_elems, ptr(y), regs, rank, world, st))

    def dx_push(self, prob, d_gate: Tensor, d_up: Tensor, w_gate: Tensor, w_up: Tensor, dx: Tensor, max_elems: int,
                regions, rank: int, world: int) -> None:
        C = self._C
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_bwd_dx_push(
                C.byref(prob), d_gate.data_ptr(), d_up.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), dx.data_ptr(),
                max_elems, (C.c_void_p * world)(*regions), rank, world,
                torch.cuda.current_stream(self.device).cuda_stream))

    def reduce_gather(self, t: Tensor, max_elems: int, regions, rank: int, world: int) -> None:
        C = self._C
        with torch.cuda.device(self.device):
            self._lib_mod.check(self.lib.gmlp_peer_reduce_gather(
                self._lib_mod.dtype_code(t.dtype), t.numel(), max_elems, t.data_ptr(), (C.c_void_p * world)(*regions),
                rank, world, torch.cuda.current_stream(self.device).cuda_stream))


class PeerAllReduce:
    """Sum of a small tensor over the tensor-parallel group through the peers' memory.

    For the partial outputs of the down projection at decode sizes (up to about 1 MB),
    where a ring all-reduce is dominated by its latency: one kernel per rank pushes its
    partial into every peer's inbox over NVLink (plain peer stores), exchanges flags and
    adds the partials in rank order, so the ranks get identical bits. Construction is
    collective over `group`: every rank allocates one peer-mappable region and maps
    everyone else's. Then, on every rank alike and on one stream:

        y = comm.all_reduce(y_partial)            # or out=y_partial for in place

    The call number lives on the device, so calls can be captured in a CUDA graph and
    replayed (by all ranks alike). The reference has no multi-GPU path; this replaces
    parallel.all_reduce_sum (NCCL) on the decode path only.
    """

    def __init__(self, group, max_elems: int, dtype: torch.dtype, device: torch.device, backend=None):
        if dtype not in (torch.bfloat16, torch.float16):
            raise NotImplementedError(f"peer all-reduce sums bfloat16 or float16 partials; got {dtype}")
        if max_elems <= 0:
            raise ValueError("max_elems must be positive")
        self.group, self.dtype, self.device = group, dtype, device
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if not 2 <= self.world <= 8:
            raise ValueError(f"peer all-reduce covers 2 to 8 ranks of one NVLink domain; group has {self.world}")
        self.backend = backend if backend is not None else _LibPeerBackend(device)
        self.max_elems = int(max_elems)
        self.region_bytes = self.backend.region_bytes(self.max_elems, self.world)
        self.local_ptr, handle = self.backend.alloc(self.region_bytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, handle, group=group)
        self.regions = [self.local_ptr if r == self.rank else self.backend.open(handles[r])
                        for r in range(self.world)]
        # Nobody may push into a region before its owner has zeroed it and everyone has mapped it.
        dist.barrier(group=group)
        self.calls = 0

    @property
    def closed(self) -> bool:
        return self.regions is None

    def supports(self, t: Tensor) -> bool:
        n = t.numel()
        return (not self.closed and t.dtype == self.dtype and t.is_contiguous()
                and 0 < n <= self.max_elems and n % 8 == 0)

    def all_reduce(self, partial: Tensor, out: Optional[Tensor] = None, dependent: bool = False) -> Tensor:
        """Sum of `partial` over the ranks, enqueued on the current stream; returns `out` (allocated if None,
        may be `partial` itself).

        `dependent=True` launches the reduction as a programmatic dependent of the
        preceding kernel on the stream, which must be the one that wrote `partial`.
        """
        if self.closed:
            raise RuntimeError("this PeerAllReduce has been closed")
        if not self.supports(partial):
            raise ValueError(
                f"partial must be a contiguous {self.dtype} tensor of a positive multiple of 8 elements, "
                f"at most {self.max_elems}; got {tuple(partial.shape)} {partial.dtype}")
        if out is None:
            out = torch.empty_like(partial)
        elif out.numel() != partial.numel() or out.dtype != self.dtype or not out.is_contiguous():
            raise ValueError("out must be a contiguous tensor of the partial's size and dtype")
        self.calls += 1
        self.backend.allreduce(self.dtype, partial.numel(), self.max_elems, partial, self.regions, self.rank,
                               self.world, out, dependent)
        return out

    def supports_down_sum(self, M: int, K: int, dtype: torch.dtype) -> bool:
        """Whether down_fwd_sum can take a partial output of M rows and K columns."""
        n = M * K
        return (not self.closed and dtype == self.dtype and M > 0 and M % (32 * self.world) == 0
                and n <= self.max_elems and n % (8 * self.world) == 0)

    def down_fwd_sum(self, h: Tensor, w_down: Tensor, b_down: Optional[Tensor] = None,
                     residual: Optional[Tensor] = None, tuning: int = 0) -> Tensor:
        """y = sum over ranks of (h W_down^T (+ b_down) (+ residual)) for tensor-parallel shards h [M, N / world],
        W_down [K, N / world]: the down projection pushes the blocks of the other ranks' rows into their inboxes
        from its own epilogue (the scatter half of a reduce-scatter, overlapped with the GEMM's remaining
        tiles); a second kernel adds each rank's rows in rank order and hands them round. Every rank of the
        group makes the call (same M); give bias and residual on one rank only. Replaces kernels.down_fwd +
        all_reduce_sum."""
        from .ops import kernels

        M, K = h.shape[0], w_down.shape[0]
        if not self.supports_down_sum(M, K, h.dtype):
            raise ValueError(f"down_fwd_sum needs M a multiple of 32 * world, M * K <= {self.max_elems} and "
                             f"{self.dtype} operands; got M={M}, K={K}, {h.dtype}")
        h, w_down = h.contiguous(), w_down.contiguous()
        y = torch.empty((M, K), dtype=h.dtype, device=h.device)
        prob = kernels._problem(M, K, h.shape[1], h.dtype, kernels.NO_DROPOUT, kernels.NO_SHARD, tuning=tuning)
        self.calls += 1
        self.backend.down_push_sum(prob, h, w_down, b_down, residual, y, self.max_elems, self.regions, self.rank,
                                   self.world)
        return y

    def dx_push(self, d_gate: Tensor, d_up: Tensor, w_gate: Tensor, w_up: Tensor, tuning: int = 0) -> Tensor:
        """This rank's partial dx = d_gate W_gate + d_up W_up with the other ranks' row blocks pushed into their
        inboxes from the GEMM's epilogue. The result is complete only after finish_sum(dx), which every rank
        enqueues later on the same stream (behind the weight-gradient GEMMs, say) with no other call on this
        object in between."""
        from .ops import kernels

        M, N = d_gate.shape
        K = w_gate.shape[1]
        if not self.supports_down_sum(M, K, d_gate.dtype):
            raise ValueError(f"dx_push needs M a multiple of 32 * world and M * K <= {self.max_elems}; got M={M}, K={K}")
        dx = torch.empty((M, K), dtype=d_gate.dtype, device=d_gate.device)
        prob = kernels._problem(M, K, N, d_gate.dtype, kernels.NO_DROPOUT, kernels.NO_SHARD, tuning=tuning)
        self.backend.dx_push(prob, d_gate.contiguous(), d_up.contiguous(), w_gate.contiguous(), w_up.contiguous(), dx,
                             self.max_elems, self.regions, self.rank, self.world)
        return dx

    def finish_sum(self, t: Tensor) -> Tensor:
        """Second half of dx_push: sum each rank's rows in rank order and hand them round, in place."""
        self.calls += 1
        self.backend.reduce_gather(t, self.max_elems, self.regions, self.rank, self.world)
        return t

    def close(self) -> None:
        """Collective: unmap the peers' regions and free this rank's (after everyone has stopped using them)."""
        if self.regions is None:
            return
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        for r, b in enumerate(self.regions):
            if r != self.rank:
                self.backend.close(b)
        dist.barrier(group=self.group)
        self.backend.free(self.local_ptr)
        self.regions = None
