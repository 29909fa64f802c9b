"""Runs the decode forward (K=8192, N=28672, bf16) a few times: the command profiled for
profiles/decode_stream_kernels_k8192_n28672.md. Usage: python tests/perf/decode_once.py [M]"""
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import __graft_entry__ as entry  # noqa: E402

pkg = entry.load_package()
K_ = pkg.ops.kernels
dev = torch.device("cuda:0")
K, N = 8192, 28672
M = int(sys.argv[1]) if len(sys.argv) > 1 else 1
g = torch.Generator(device=dev).manual_seed(0)
wg, wu = (torch.randn((N, K), device=dev, dtype=torch.bfloat16, generator=g) * 0.02 for _ in range(2))
wd = torch.randn((K, N), device=dev, dtype=torch.bfloat16, generator=g) * 0.02
x = torch.randn((M, K), device=dev, dtype=torch.bfloat16, generator=g)
scratch = K_.decode_scratch(M, K, N, torch.bfloat16, dev)
for _ in range(4):
    K_.decode_fwd(x, wg, None, wu, None, wd, None, scratch=scratch)
torch.cuda.synchronize()
n = 20
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for _ in range(n):
    K_.decode_fwd(x, wg, None, wu, None, wd, None, scratch=scratch)
e1.record()
torch.cuda.synchronize()
us = e0.elapsed_time(e1) / n * 1e3
nbytes = 2 * (3 * K * N + 2 * M * K)
print(f"decode M={M}: {us:.1f} us per forward, {nbytes / us / 1e3:.0f} GB/s algorithmic")
assert pkg._lib.status_read(dev) == 0
