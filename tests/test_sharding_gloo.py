"""world_size-2 CPU ranks (gloo): the sharding arithmetic and the collectives of the
two multi-GPU modes, with the CPU oracle standing in for the kernels."""
import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
WORLD = 2


class _FakePeerBackend:
    """Stands in for the CUDA IPC + kernel side of PeerAllReduce: recorded calls, no device."""

    def __init__(self, rank):
        self.rank, self.launches, self.closed, self.freed = rank, [], [], []

    def region_bytes(self, max_elems, world):
        return 2 * world * max_elems * 2 + 4096

    def alloc(self, nbytes):
        self.nbytes = nbytes
        return 0x7000 + self.rank, bytes([self.rank]) * 64

    def open(self, handle):
        return 0x10000000 * (handle[0] + 1)

    def allreduce(self, dtype, n, max_elems, src, regions, rank, world, dst, dependent):
        self.launches.append((n, max_elems, src.data_ptr(), list(regions), rank, world, dst.data_ptr(), dependent))

    def down_push_sum(self, prob, h, w_down, b_down, residual, y, max_elems, regions, rank, world):
        self.launches.append(("down_push_sum", prob.M, prob.K, prob.N, y.data_ptr(), max_elems, rank, world))

    def dx_push(self, prob, d_gate, d_up, w_gate, w_up, dx, max_elems, regions, rank, world):
        self.launches.append(("dx_push", prob.M, prob.K, prob.N, dx.data_ptr(), max_elems, rank, world))

    def reduce_gather(self, t, max_elems, regions, rank, world):
        self.launches.append(("reduce_gather", t.numel(), t.data_ptr(), max_elems, rank, world))

    def close(self, ptr):
        self.closed.append(ptr)

    def free(self, ptr):
        self.freed.append(ptr)


def _peer_host_logic(P, rank):
    """Handle exchange, argument checks and teardown of PeerAllReduce (no GPU involved)."""
    fake = _FakePeerBackend(rank)
    comm = P.PeerAllReduce(dist.group.WORLD, 64 * 24, torch.bfloat16, torch.device("cpu"), backend=fake)
    other = 1 - rank
    assert fake.nbytes == fake.region_bytes(64 * 24, WORLD)
    assert comm.regions[rank] == 0x7000 + rank and comm.regions[other] == 0x10000000 * (other + 1)
    part = torch.zeros((8, 24), dtype=torch.bfloat16)
    out = comm.all_reduce(part, dependent=True)
    assert out.shape == (8, 24) and out.data_ptr() != part.data_ptr()
    assert fake.launches[-1] == (192, 64 * 24, part.data_ptr(), comm.regions, rank, WORLD, out.data_ptr(), True)
    assert comm.all_reduce(part, out=part) is part            # in place
    assert fake.launches[-1][2] == fake.launches[-1][6] == part.data_ptr() and comm.calls == 2
    for bad in (torch.zeros((65, 24), dtype=torch.bfloat16),     # more than max_elems
                torch.zeros((1, 12), dtype=torch.bfloat16),      # not a multiple of 8 elements
                torch.zeros((8, 24), dtype=torch.float16),       # not the group's dtype
                torch.zeros((8, 48), dtype=torch.bfloat16)[:, ::2]):   # not contiguous
        assert not comm.supports(bad)
        with pytest.raises(ValueError):
            comm.all_reduce(bad)
    with pytest.raises(ValueError):
        comm.all_reduce(part, out=torch.zeros((4, 24), dtype=torch.bfloat16))
    # the pushing GEMMs: rows must split into 32-row blocks per rank and fit the regions
    bf = torch.bfloat16
    big = P.PeerAllReduce(dist.group.WORLD, 128 * 24, bf, torch.device("cpu"), backend=_FakePeerBackend(rank))
    assert big.supports_down_sum(128, 24, bf) and big.supports_down_sum(64, 24, bf)
    assert not big.supports_down_sum(96, 24, bf)          # 96 rows are not a multiple of 32 * world
    assert not big.supports_down_sum(256, 24, bf)         # above the capacity
    assert not big.supports_down_sum(128, 24, torch.float16)
    y = big.down_fwd_sum(torch.zeros((128, 40), dtype=bf), torch.zeros((24, 40), dtype=bf))
    assert y.shape == (128, 24)
    assert big.backend.launches[-1] == ("down_push_sum", 128, 24, 40, y.data_ptr(), 128 * 24, rank, WORLD)
    dx = big.dx_push(torch.zeros((64, 40), dtype=bf), torch.zeros((64, 40), dtype=bf),
                     torch.zeros((40, 24), dtype=bf), torch.zeros((40, 24), dtype=bf))
    assert dx.shape == (64, 24) and big.backend.launches[-1][:4] == ("dx_push", 64, 24, 40)
    assert big.finish_sum(dx) is dx
    assert big.backend.launches[-1] == ("reduce_gather", 64 * 24, dx.data_ptr(), 128 * 24, rank, WORLD)
    with pytest.raises(ValueError):
        big.down_fwd_sum(torch.zeros((96, 40), dtype=bf), torch.zeros((24, 40), dtype=bf))
    big.close()
    comm.close()
    assert fake.closed == [0x10000000 * (other + 1)] and fake.freed == [0x7000 + rank]
    comm.close()                                              # idempotent
    assert comm.closed and not comm.supports(part)            # callers fall back to NCCL after close()
    with pytest.raises(RuntimeError):
        comm.all_reduce(part)


def _worker(rank, port, mode, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import __graft_entry__ as entry
    from oracle import gated_mlp_oracle as orc

    pkg = entry.load_package()
    P = pkg.parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        M, K, N = 48, 32, 64
        p, seed, offset = 0.25, 99, 4
        case = orc.make_case(M, K, N, True, torch.bfloat16, seed=1, w_std=0.2)
        want = orc.forward_backward(case, dropout_p=p, seed=seed, offset=offset)
        x, wg, bg, wu, bu, wd, bd, dy = case.f32()
        if mode == "tp":
            sd = P.shard_tp_state_dict(case.state_dict(), rank, WORLD)
            c0, cols = P.tp_shard_range(N, rank, WORLD)
            mod = pkg.FusedGatedMLP(K, cols, parallel_mode="tp")   # reads rank/size from the group
            s = mod._shard()
            assert (s.col0, s.n_global) == (c0, N)
            ks = orc.keep_scale_tensor(M, cols, p, seed, offset, col0=s.col0, n_global=s.n_global)
            y = orc.forward(x, sd["gate_proj.weight"], sd["gate_proj.bias"], sd["up_proj.weight"],
                            sd["up_proj.bias"], sd["down_proj.weight"], bd if rank == 0 else None, ks)
            P.all_reduce_sum(y, dist.group.WORLD)
            g = orc.backward(x, sd["gate_proj.weight"], sd["gate_proj.bias"], sd["up_proj.weight"],
                             sd["up_proj.bias"], sd["down_proj.weight"], bd, dy, ks)
            P.all_reduce_sum(g["dx"], dist.group.WORLD)
            full = P.gather_tp_grads({k[1:]: v for k, v in g.items() if k != "dx"})
            torch.testing.assert_close(y, want["y"], rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(g["dx"], want["dx"], rtol=1e-4, atol=1e-5)
            for k, v in full.items():
                torch.testing.assert_close(v, want["d" + k], rtol=1e-4, atol=1e-5)
        elif mode == "peer":
            _peer_host_logic(P, rank)
        elif mode == "overlap":
            # chunked partial sums with the all-reduce of chunk i started before chunk i+1 is produced
            assert P.chunk_ranges(10, 4) == [(0, 4), (4, 8), (8, 10)] and P.chunk_ranges(10, 0) == [(0, 10)]
            assert P.chunk_ranges(10, 10) == [(0, 10)] and P.chunk_ranges(0, 4) == []
            sd = P.shard_tp_state_dict(case.state_dict(), rank, WORLD)
            h = orc.hidden_forward(x, sd["gate_proj.weight"], sd["gate_proj.bias"], sd["up_proj.weight"],
                                   sd["up_proj.bias"])[0]
            y = torch.empty((M, K))
            log = []

            def produce(r0, r1):
                log.append(("rows", r0, r1))
                y[r0:r1] = h[r0:r1] @ sd["down_proj.weight"].T + (bd if rank == 0 else 0.0)

            works = P.overlapped_all_reduce(y, produce, dist.group.WORLD, 20, lambda on: log.append(("limit", on)))
            assert log == [("rows", 0, 20), ("limit", True), ("rows", 20, 40), ("rows", 40, 48)] and len(works) == 3
            P.wait_all(works)
            torch.testing.assert_close(y, orc.forward_backward(case, grads=False)["y"], rtol=1e-4, atol=1e-5)
        else:
            r0, rows = P.token_shard_range(M, rank, WORLD)
            ks = orc.keep_scale_tensor(rows, N, p, seed, offset, row0=r0)
            xs, dys = x[r0:r0 + rows], dy[r0:r0 + rows]
            y = orc.forward(xs, wg, bg, wu, bu, wd, bd, ks)
            g = orc.backward(xs, wg, bg, wu, bu, wd, bd, dys, ks)
            torch.testing.assert_close(y, want["y"][r0:r0 + rows], rtol=1e-4, atol=1e-5)
            torch.testing.assert_close(g["dx"], want["dx"][r0:r0 + rows], rtol=1e-4, atol=1e-5)
            # weight gradients are rank-local partial sums: their sum is the full gradient
            for k in ("dgate_proj.weight", "ddown_proj.weight", "dup_proj.bias"):
                t = g[k].clone()
                dist.all_reduce(t)
                torch.testing.assert_close(t, want[k], rtol=1e-4, atol=1e-5)
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["tp", "token", "peer", "overlap"])
def test_two_rank_sharding(mode):
    port = 29500 + (os.getpid() % 2000) + {"tp": 0, "token": 1, "peer": 2, "overlap": 3}[mode]
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(port, mode, ret), nprocs=WORLD, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}
