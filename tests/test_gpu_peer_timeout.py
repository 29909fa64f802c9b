"""Failure detection of the peer all-reduce without a second process: a rank whose peer never
shows up gives up its bounded wait, reports it through the status word and leaves the context
usable; the peer, arriving later, still finds the first rank's data and completes.

Both "ranks" are plain buffers on one GPU and their kernels run one after the other, so nothing
here waits on a concurrently running kernel."""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_missing_peer_times_out_and_late_peer_completes(pkg, cuda_dev):
    L = pkg._lib
    lib = L.load()
    n, world = 1024, 2
    nbytes = lib.gmlp_peer_region_bytes(n, world)
    assert nbytes > 2 * world * n * 2
    regions = []
    with torch.cuda.device(cuda_dev):
        for _ in range(world):
            p, handle = C.c_void_p(), C.create_string_buffer(64)
            L.check(lib.gmlp_peer_alloc(nbytes, C.byref(p), handle))
            regions.append(p.value)
    try:
        arr = (C.c_void_p * world)(*regions)
        stream = torch.cuda.current_stream(cuda_dev).cuda_stream
        src0 = torch.full((n,), 1.5, dtype=torch.bfloat16, device=cuda_dev)
        src1 = torch.full((n,), 2.25, dtype=torch.bfloat16, device=cuda_dev)
        dst0 = torch.full((n,), 7.0, dtype=torch.bfloat16, device=cuda_dev)
        dst1 = torch.full((n,), 7.0, dtype=torch.bfloat16, device=cuda_dev)
        torch.cuda.synchronize()

        # rank 0 alone: nobody raises rank 1's flag
        t0 = time.perf_counter()
        with torch.cuda.device(cuda_dev):
            L.check(lib.gmlp_peer_allreduce(L.GMLP_BF16, n, n, src0.data_ptr(), arr, 0, world, dst0.data_ptr(), 0,
                                            stream))
        status = L.status_read(cuda_dev)                      # synchronises the device
        waited = time.perf_counter() - t0
        assert status == 4, f"status {status}: the wait for the missing peer should have run out"
        assert 0.2 < waited < 20.0, f"the bounded wait took {waited:.2f} s"
        assert torch.equal(dst0, torch.full_like(dst0, 7.0)), "dst must be left unwritten after a timeout"
        assert L.status_read(cuda_dev) == 0                   # read once, cleared

        # the context is intact: an ordinary kernel still runs and is right
        a = torch.randn((128, 64), device=cuda_dev).to(torch.bfloat16)
        b = torch.randn((256, 64), device=cuda_dev).to(torch.bfloat16)
        c = pkg.ops.kernels.gemm(a, b)
        assert (c.float() - a.float() @ b.float().T).abs().max().item() < 0.25

        # rank 1 arrives late (its first call too): rank 0's partial and flag are already in its
        # region, so it does not wait and gets the full sum
        with torch.cuda.device(cuda_dev):
            L.check(lib.gmlp_peer_allreduce(L.GMLP_BF16, n, n, src1.data_ptr(), arr, 1, world, dst1.data_ptr(), 0,
                                            stream))
        assert L.status_read(cuda_dev) == 0
        assert torch.equal(dst1, torch.full_like(dst1, 3.75))
    finally:
        torch.cuda.synchronize()
        with torch.cuda.device(cuda_dev):
            for p in regions:
                L.check(lib.gmlp_peer_free(p))


def test_peer_allreduce_argument_checks(pkg, cuda_dev):
    L = pkg._lib
    lib = L.load()
    t = torch.zeros(64, dtype=torch.bfloat16, device=cuda_dev)
    arr = (C.c_void_p * 2)(t.data_ptr(), t.data_ptr())
    with torch.cuda.device(cuda_dev):
        assert lib.gmlp_peer_allreduce(L.GMLP_BF16, 12, 64, t.data_ptr(), arr, 0, 2, t.data_ptr(), 0, None) == -1
        assert lib.gmlp_peer_allreduce(L.GMLP_BF16, 128, 64, t.data_ptr(), arr, 0, 2, t.data_ptr(), 0, None) == -1
        assert lib.gmlp_peer_allreduce(L.GMLP_BF16, 64, 64, t.data_ptr(), arr, 2, 2, t.data_ptr(), 0, None) == -6
        assert lib.gmlp_peer_allreduce(L.GMLP_BF16, 64, 64, t.data_ptr(), arr, 0, 9, t.data_ptr(), 0, None) == -6
        assert lib.gmlp_peer_allreduce(7, 64, 64, t.data_ptr(), arr, 0, 2, t.data_ptr(), 0, None) == -3
        assert lib.gmlp_peer_allreduce(L.GMLP_BF16, 64, 64, None, arr, 0, 2, t.data_ptr(), 0, None) == -6
    assert lib.gmlp_peer_region_bytes(0, 2) == 0 and lib.gmlp_peer_region_bytes(64, 9) == 0
    assert b"rank" in lib.gmlp_last_error() or len(lib.gmlp_last_error()) > 0
