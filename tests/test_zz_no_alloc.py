"""gmlp_colsum_static: the column-sum entry point for hosts that cannot allocate.

Some hosts of this library hand every byte of device memory to their own pool when
they start and have no allocator to ask for scratch afterwards (and no torch); others
sit in a latency-critical loop where an allocation's device-wide synchronisation is
not acceptable. For them the library keeps 1 MiB of scratch in its own image. This
test calls that entry point through the C ABI, twice in a row on different data, and
holds it to the result of the ordinary gmlp_colsum (caller-provided scratch).

The file name sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_colsum(pkg, src, dst=None):
    L = pkg._lib
    if dst is None:
        dst = torch.empty((src.shape[1],), dtype=src.dtype, device=src.device)
    with torch.cuda.device(src.device):
        rc = L.load().gmlp_colsum_static(src.shape[0], src.shape[1], L.dtype_code(src.dtype), src.data_ptr(),
                                         src.stride(0), dst.data_ptr(),
                                         torch.cuda.current_stream(src.device).cuda_stream)
    return rc, dst


def _alloc_state(dev):
    """What an allocation anywhere would move: the driver's free-memory figure and torch's allocator counters."""
    torch.cuda.synchronize(dev)
    free, _ = torch.cuda.mem_get_info(dev)
    st = torch.cuda.memory_stats(dev)
    return free, st.get("allocation.all.allocated", 0), st.get("segment.all.allocated", 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_static_scratch_matches_caller_scratch_twice(pkg, cuda_dev, dtype):
    g = torch.Generator(device=cuda_dev).manual_seed(17)
    shapes = [(4096, 2048), (777, 8192)]       # two calls in a row; the second reuses the array
    for rows, cols in shapes:
        src = (torch.randn((rows, cols), device=cuda_dev, generator=g) * 0.1).to(dtype)
        want = pkg.ops.kernels.colsum(src)     # existing entry point, torch-allocated scratch
        rc, got = _static_colsum(pkg, src)
        assert rc == 0, pkg._lib.load().gmlp_last_error()
        torch.cuda.synchronize()
        # same kernels, same partition of the rows: the results are identical, which is
        # stricter than the 2e-2 / 1e-2 parity tolerance used elsewhere
        assert torch.equal(got, want)
        ref = src.float().sum(0)
        assert (got.float() - ref).abs().max().item() <= 2e-2 * max(1.0, ref.pow(2).mean().sqrt().item())


def test_static_scratch_call_allocates_nothing(pkg, cuda_dev):
    """The property in the entry point's name: across the call neither the driver's free memory nor torch's
    allocator statistics move. Source and destination exist before the window opens, and the first call on
    the device (which loads the library image and looks the array up) is made outside it."""
    src = (torch.randn((2048, 1024), device=cuda_dev) * 0.1).to(torch.bfloat16)
    dst = torch.empty((1024,), dtype=torch.bfloat16, device=cuda_dev)
    rc, _ = _static_colsum(pkg, src, dst)
    assert rc == 0
    before = _alloc_state(cuda_dev)
    for _ in range(3):
        rc, _ = _static_colsum(pkg, src, dst)
        assert rc == 0
    assert _alloc_state(cuda_dev) == before
    assert (dst.float() - src.float().sum(0)).abs().max().item() <= 2e-2 * max(1.0, src.float().sum(0).std().item())


@pytest.mark.parametrize("rows,cols,ld", [(40, 256, 256), (4096, 512, 1536), (63, 128, 384)])
def test_static_scratch_strided_source_and_few_rows(pkg, cuda_dev, rows, cols, ld):
    """A source that is a column slice of a wider matrix (row pitch > cols), and fewer than 64 rows (a single
    row block): same answer as the caller-scratch entry point."""
    g = torch.Generator(device=cuda_dev).manual_seed(rows + cols)
    wide = (torch.randn((rows, ld), device=cuda_dev, generator=g) * 0.1).to(torch.bfloat16)
    src = wide[:, :cols]
    assert src.stride(0) == ld
    rc, got = _static_colsum(pkg, src)
    assert rc == 0, pkg._lib.load().gmlp_last_error()
    want = pkg.ops.kernels.colsum(src.contiguous())
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_static_scratch_refuses_what_does_not_fit(pkg, cuda_dev):
    cols = (1 << 18) + 8                       # 4 * cols bytes of partial sums already exceed 1 MiB
    src = torch.zeros((64, cols), dtype=torch.bfloat16, device=cuda_dev)
    rc, _ = _static_colsum(pkg, src)
    assert rc == -7
    msg = pkg._lib.load().gmlp_last_error().decode()
    assert "built-in scratch" in msg and "gmlp_colsum" in msg
