"""Tensor-parallel decode forward (K=8192, N=28672 split over the ranks, bf16): time per step with
the partial outputs summed by NCCL and by the one-shot peer-memory kernel, and the two sums alone
(all from CUDA graphs, so that the device time is measured and not the host's launch rate).
Usage: python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
       --master-port 29650 tests/perf/tp_decode.py [nodep]"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import __graft_entry__ as entry  # noqa: E402


def timed(fn, dev, inner=20, reps=10):
    """Milliseconds per call of `fn` on the device: `inner` calls captured in one CUDA graph (so the host's
    launch cost is out of the picture), `reps` replays timed with events, max over ranks."""
    side = torch.cuda.Stream(dev)
    side.wait_stream(torch.cuda.current_stream(dev))
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(inner):
                fn()
    torch.cuda.current_stream(dev).wait_stream(side)
    graph.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / (reps * inner)], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    K, N = 8192, 28672
    cols = N // world
    torch.manual_seed(rank)
    try:
        m = pkg.FusedGatedMLP(K, cols, bias=False, parallel_mode="tp").to(dev).to(torch.bfloat16).eval()
        for q in m.parameters():
            q.data.normal_(0, 0.02)
        rows = []
        hook = pkg._lib.load().gmlp_set_peer_two_shot_bytes
        for M in (1, 8, 32, 64):
            x = torch.randn((M, K), device=dev, dtype=torch.bfloat16)
            y = torch.empty((M, K), device=dev, dtype=torch.bfloat16)
            with torch.no_grad():
                m._peer = None
                t_nccl = timed(lambda: m(x), dev)
                t_ar_nccl = timed(lambda: dist.all_reduce(y), dev)
                comm = m.enable_peer_allreduce(64)
                m.peer_max_bytes = 1 << 30   # time the peer sum at every M, also above the module's default cap
                if "nodep" in sys.argv:      # the peer sum as an ordinary launch, not a programmatic dependent
                    plain = comm.all_reduce
                    comm.all_reduce = lambda t, out=None, dependent=False: plain(t, out=out, dependent=False)
                t_peer = timed(lambda: m(x), dev)
                hook(-1)   # every partial to every peer
                t_ar_one = timed(lambda: comm.all_reduce(y, out=y), dev)
                hook(1)    # slices reduced by their owners
                t_ar_two = timed(lambda: comm.all_reduce(y, out=y), dev) if y.numel() % (8 * world) == 0 else float("nan")
                hook(0)
                comm.close()
            rows.append((M, t_nccl, t_peer, t_ar_nccl, t_ar_one, t_ar_two))
        assert pkg._lib.status_read(dev) == 0
        if rank == 0:
            for M, a, b, c, d, e in rows:
                print(f"tp{world} decode M={M}: step {a * 1e3:.1f} us with NCCL sum, {b * 1e3:.1f} us with peer sum; "
                      f"sum alone {c * 1e3:.1f} us NCCL, {d * 1e3:.1f} us peer one-shot, {e * 1e3:.1f} us peer two-shot",
                      flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
