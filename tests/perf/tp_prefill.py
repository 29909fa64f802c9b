"""Tensor-parallel prefill / training step (K=8192, N=28672 split over the ranks, bf16, M rows replicated):
time per forward and per forward+backward with one all-reduce after the whole GEMM against the chunked form
(module.tp_chunk_rows_fwd, module.tp_chunk_rows) whose all-reduces overlap the next chunk's GEMM.
Usage: python -m torch.distributed.run --nnodes=1 --nproc-per-node G --master-addr 127.0.0.1 \
       --master-port 29651 tests/perf/tp_prefill.py [M]"""
import os
import sys
from pathlib import Path

os.environ.setdefault("NCCL_MAX_CTAS", "16")  # the collective's CTAs must fit into the SMs the GEMMs leave free

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import __graft_entry__ as entry  # noqa: E402


def timed(fn, n, dev):
    """Milliseconds per call, max over ranks (device events, barrier on both sides)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    M = int(sys.argv[1]) if len(sys.argv) > 1 else 16384
    K, N = 8192, 28672
    cols = N // world
    torch.manual_seed(rank)
    try:
        m = pkg.FusedGatedMLP(K, cols, bias=False, parallel_mode="tp").to(dev).to(torch.bfloat16)
        for q in m.parameters():
            q.data.normal_(0, 0.01)
        x = torch.randn((M, K), device=dev, dtype=torch.bfloat16, requires_grad=True)
        dy = torch.randn((M, K), device=dev, dtype=torch.bfloat16) * 1e-2

        def fwd():
            with torch.no_grad():
                m(x)

        def fwd_bwd():
            m(x).backward(dy)
            m.zero_grad(set_to_none=True)
            x.grad = None

        rows = []
        # (forward chunk rows, backward chunk rows, SMs left to the collective)
        for cf, cb, sms in ((0, 0, 16), (0, 4096, 16), (4096, 4096, 16), (0, 2048, 16), (0, 4096, 32)):
            m.tp_chunk_rows_fwd, m.tp_chunk_rows, m.tp_comm_sms = cf, cb, sms
            rows.append((f"{cf}/{cb}", sms, timed(fwd, 10, dev), timed(fwd_bwd, 5, dev)))
        assert pkg._lib.status_read(dev) == 0
        if rank == 0:
            for chunk, sms, tf, tb in rows:
                pf = 6.0 * M * K * N / tf / 1e12          # whole-job PFLOP/s (N is the un-sharded size)
                pb = 18.0 * M * K * N / tb / 1e12
                print(f"tp{world} M={M} chunk_rows(fwd/bwd)={chunk} comm_sms={sms}: fwd {tf:.3f} ms ({pf:.2f} PFLOP/s), "
                      f"fwd+bwd {tb:.3f} ms ({pb:.2f} PFLOP/s)", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
