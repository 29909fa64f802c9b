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

from typing import Dict, Optional, Tuple

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
