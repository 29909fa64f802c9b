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


@pytest.mark.parametrize("mode", ["tp", "token"])
def test_two_rank_sharding(mode):
    port = 29500 + (os.getpid() % 2000) + (0 if mode == "tp" else 1)
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(port, mode, ret), nprocs=WORLD, join=True)
        assert dict(ret) == {0: "ok", 1: "ok"}
