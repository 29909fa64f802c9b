"""Worker for tests/test_gpu_multi.py: one process per GPU (launched by torch.distributed.run).

Checks the two sharded modes of FusedGatedMLP on real GPUs over NCCL against the
single-process CPU oracle: tensor parallel (intermediate dimension sharded, y and dx
all-reduced) for training and for the decode path, and token sharding (no collective,
dropout mask offset by the shard's first global row).
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402
from oracle import gated_mlp_oracle as orc  # noqa: E402


def main():
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    pkg = entry.load_package()
    P = pkg.parallel
    dt = torch.bfloat16
    try:
        # ---------------- tensor parallel, training step with bias and dropout
        M, K, N = 384, 256, 128 * world * 2
        p, seed, offset = 0.1, 77, 5
        case = orc.make_case(M, K, N, True, dt, seed=11, w_std=0.5 * K ** -0.5, dy_std=0.05)
        want = orc.forward_backward(case, dropout_p=p, seed=seed, offset=offset)
        c0, cols = P.tp_shard_range(N, rank, world)
        m = pkg.FusedGatedMLP(K, cols, bias=True, dropout_p=p, parallel_mode="tp")
        m.load_state_dict(P.shard_tp_state_dict(case.state_dict(), rank, world))
        m = m.to(dev).to(dt).train()
        m.set_philox(seed, offset)
        x = case.x.to(dev).requires_grad_(True)
        y = m(x)
        y.backward(case.dy.to(dev))
        orc.assert_parity(y.cpu(), want["y"], "tp y")
        orc.assert_parity(x.grad.cpu(), want["dx"], "tp dx")
        full = P.gather_tp_grads({n: q.grad for n, q in m.named_parameters()})
        for n, g in full.items():
            orc.assert_parity(g.cpu(), want["d" + n], "tp d" + n)

        # ---------------- the same step with the down projection and dx computed in chunks of 128 rows,
        # each chunk's all-reduce overlapping the next chunk's GEMM
        m.tp_chunk_rows = m.tp_chunk_rows_fwd = 128
        m.zero_grad(set_to_none=True)
        m.set_philox(seed, offset)
        x2 = case.x.to(dev).requires_grad_(True)
        y2 = m(x2)
        y2.backward(case.dy.to(dev))
        orc.assert_parity(y2.cpu(), want["y"], "tp y (chunked)")
        orc.assert_parity(x2.grad.cpu(), want["dx"], "tp dx (chunked)")
        full2 = P.gather_tp_grads({n: q.grad for n, q in m.named_parameters()})
        for n, g in full2.items():
            assert torch.equal(g, full[n]), f"chunking changed d{n}"
        assert pkg._lib.set_sm_limit(0) == 0, "the SM limit must be back to 0 after a chunked step"

        # ---------------- tensor parallel, decode path (M <= 64, no grad)
        Md, Kd, Nd = 8, 512, 256 * world
        cased = orc.make_case(Md, Kd, Nd, True, dt, seed=12, w_std=0.5 * Kd ** -0.5)
        _, colsd = P.tp_shard_range(Nd, rank, world)
        md = pkg.FusedGatedMLP(Kd, colsd, bias=True, parallel_mode="tp")
        md.load_state_dict(P.shard_tp_state_dict(cased.state_dict(), rank, world))
        md = md.to(dev).to(dt).eval()
        with torch.no_grad():
            yd = md(cased.x.to(dev))
        assert md._decode_scratch is not None
        orc.assert_parity(yd.cpu(), orc.forward_backward(cased, grads=False)["y"], "tp decode y")

        # ---------------- one-shot sum over peer memory: bit-exact against the rank-ordered fp32 sum,
        # many calls in flight (no host synchronisation between them: the two inbox parities
        # and the epoch flags alone keep the ranks apart), out of place and in place
        comm = P.PeerAllReduce(dist.group.WORLD, 64 * 8192, dt, dev)
        # up to 128 KB: every partial pushed to every peer; from 256 KB: slices reduced by their owners
        shapes = ((1, 8), (8, 512), (64, 1024), (3, 1000), (40, 4096), (64, 8192))
        cases = []
        for shape in shapes:
            gen = torch.Generator().manual_seed(1000 + shape[1])
            steps = 24 if shape[0] * shape[1] <= 65536 else 6
            vals = torch.randn((steps, world) + shape, generator=gen).to(dt)      # every rank's partials
            acc = torch.zeros((steps,) + shape)
            for r in range(world):                                                # rank order, fp32
                acc += vals[:, r].float()
            cases.append((shape, steps, vals[:, rank].to(dev), acc.to(dt)))
        pkg._lib.load().gmlp_set_peer_two_shot_bytes(256 * 1024)   # also with two ranks, where the default is one-shot
        for shape, steps, mine, want_sum in cases:
            outs = []
            for it in range(steps):
                if it % 2:
                    buf = mine[it].clone()
                    outs.append(comm.all_reduce(buf, out=buf))
                else:
                    outs.append(comm.all_reduce(mine[it]))
            got = torch.stack(outs).cpu()
            assert torch.equal(got.view(torch.int16), want_sum.view(torch.int16)), f"peer all-reduce {shape}"
        # the two forms and all sizes interleaved, still without host synchronisation
        outs = [comm.all_reduce(cases[it % len(cases)][2][it % 6]) for it in range(30)]
        for it, o in enumerate(outs):
            want_it = cases[it % len(cases)][3][it % 6]
            assert torch.equal(o.cpu().view(torch.int16), want_it.view(torch.int16)), f"interleaved call {it}"
        pkg._lib.load().gmlp_set_peer_two_shot_bytes(0)

        # the same calls captured once in a CUDA graph and replayed: the call number lives on the device
        shape = (16, 512)
        gen = torch.Generator().manual_seed(4242)
        vals = torch.randn((2, world) + shape, generator=gen).to(dt)
        src = [vals[i, rank].to(dev) for i in range(2)]
        dst = [torch.empty(shape, dtype=dt, device=dev) for _ in range(2)]
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            comm.all_reduce(src[0], out=dst[0])     # warm-up outside the capture, on every rank alike
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                comm.all_reduce(src[0], out=dst[0])
                comm.all_reduce(src[1], out=dst[1])
                comm.all_reduce(src[0], out=dst[0])
        torch.cuda.current_stream(dev).wait_stream(side)
        for _ in range(5):
            graph.replay()
        for i in range(2):
            want_i = sum(vals[i, r].float() for r in range(world)).to(dt)
            assert torch.equal(dst[i].cpu().view(torch.int16), want_i.view(torch.int16)), "peer all-reduce replay"

        # ---------------- the decode path with the peer sum chained to the down projection
        y_nccl = yd.clone()
        md.enable_peer_allreduce(max_tokens=64)
        with torch.no_grad():
            for it in range(4):
                yp = md(cased.x.to(dev))
        orc.assert_parity(yp.cpu(), orc.forward_backward(cased, grads=False)["y"], "tp decode y (peer sum)")
        assert (yp.float() - y_nccl.float()).abs().max().item() <= 2e-2
        every = [torch.empty_like(yp) for _ in range(world)]
        dist.all_gather(every, yp)
        assert all(torch.equal(e, every[0]) for e in every), "ranks disagree on the summed output"
        md.peer_max_bytes = 0                 # above the cap the module goes back to the NCCL sum
        with torch.no_grad():
            assert torch.equal(md(cased.x.to(dev)), y_nccl)
        md._peer.close()
        comm.close()
        with torch.no_grad():
            y_back = md(cased.x.to(dev))      # a closed peer group: the module is back on the NCCL sum
        assert torch.equal(y_back, y_nccl)

        # ---------------- prefill / training forward whose down projection scatters its partial output into
        # the owners' inboxes from its epilogue (no NCCL call in the forward pass)
        Mp, Kp, Np = 512, 512, 256 * world
        casep = orc.make_case(Mp, Kp, Np, True, dt, seed=14, w_std=0.5 * Kp ** -0.5, dy_std=0.05)
        wantp = orc.forward_backward(casep)
        _, colsp = P.tp_shard_range(Np, rank, world)
        mp = pkg.FusedGatedMLP(Kp, colsp, bias=True, parallel_mode="tp")
        mp.load_state_dict(P.shard_tp_state_dict(casep.state_dict(), rank, world))
        mp = mp.to(dev).to(dt).eval()
        xp = casep.x.to(dev)
        with torch.no_grad():
            y_ref = mp(xp)                                   # NCCL sum
        mp.enable_peer_output_sum(max_tokens=Mp)
        with torch.no_grad():
            ys = [mp(xp) for _ in range(6)]                  # back to back, no host synchronisation
            y_half = mp(xp[:256])                            # fewer rows than the capacity
        assert all(torch.equal(ys[0], t) for t in ys[1:]), "the pushed sum is not repeatable"
        orc.assert_parity(ys[0].cpu(), wantp["y"], "tp y (pushed sum)")
        orc.assert_parity(y_half.cpu(), wantp["y"][:256], "tp y (pushed sum, 256 rows)")
        assert (ys[0].float() - y_ref.float()).abs().max().item() <= 4e-2
        every = [torch.empty_like(ys[0]) for _ in range(world)]
        dist.all_gather(every, ys[0])
        assert all(torch.equal(e, every[0]) for e in every), "ranks disagree on the pushed sum"
        mp.train()
        xg = casep.x.to(dev).requires_grad_(True)
        yg = mp(xg)
        yg.backward(casep.dy.to(dev))
        assert torch.equal(yg.detach(), ys[0])
        orc.assert_parity(xg.grad.cpu(), wantp["dx"], "tp dx (after a pushed forward)")
        fullp = P.gather_tp_grads({n: q.grad for n, q in mp.named_parameters()})
        for n, g in fullp.items():
            orc.assert_parity(g.cpu(), wantp["d" + n], "tp d" + n + " (after a pushed forward)")
        with torch.no_grad():
            y_odd = mp.eval()(xp[:96])                       # 96 rows do not split into 32-row blocks per rank
        orc.assert_parity(y_odd.cpu(), wantp["y"][:96], "tp y (NCCL fallback)")
        torch.cuda.synchronize()
        assert pkg._lib.status_read(dev) == 0
        mp._peer_sum.close()

        # ---------------- token sharding: no collective, mask rows offset
        Mt = 256 * world
        caset = orc.make_case(Mt, K, 512, False, dt, seed=13, w_std=0.5 * K ** -0.5, dy_std=0.05)
        wantt = orc.forward_backward(caset, dropout_p=0.25, seed=seed, offset=offset)
        r0, rows = P.token_shard_range(Mt, rank, world)
        mt = pkg.FusedGatedMLP(K, 512, bias=False, dropout_p=0.25, parallel_mode="token")
        mt.load_state_dict(caset.state_dict())
        mt = mt.to(dev).to(dt).train()
        mt.set_philox(seed, offset)
        mt.token_row0 = r0
        xt = caset.x[r0:r0 + rows].to(dev).requires_grad_(True)
        yt = mt(xt)
        yt.backward(caset.dy[r0:r0 + rows].to(dev))
        orc.assert_parity(yt.cpu(), wantt["y"][r0:r0 + rows], "token y")
        orc.assert_parity(xt.grad.cpu(), wantt["dx"][r0:r0 + rows], "token dx")
        gw = mt.gate_proj.weight.grad.float()
        dist.all_reduce(gw)  # un-timed check only: rank-local partial sums add up to the full gradient
        orc.assert_parity(gw.cpu(), wantt["dgate_proj.weight"], "token dW_gate (summed over ranks)")

        torch.cuda.synchronize()
        assert pkg._lib.status_read(dev) == 0
        dist.barrier()
        if rank == 0:
            print("MULTI_GPU_OK", world, flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
