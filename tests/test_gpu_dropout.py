"""The device dropout mask must equal the CPU restatement bit for bit."""
import numpy as np
import pytest
import torch

from oracle import philox

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,N,p,seed,offset,row0,col0,ng", [
    (128, 256, 0.1, 0x5EED, 0, 0, 0, 0),
    (200, 136, 0.5, 123456789012345, 77, 0, 0, 0),
    (64, 128, 0.25, 3, 9, 4096, 128, 512),            # a token- and column-shifted shard
    (8, 1024, 0.9, 2 ** 63 + 5, 2 ** 40 + 1, 2 ** 26, 0, 1024),  # 64-bit seed/offset, index >> 3 beyond 2**32
])
def test_mask_bit_exact(pkg, cuda_dev, M, N, p, seed, offset, row0, col0, ng):
    K = pkg.ops.kernels
    got = K.dropout_mask(M, N, K.Dropout(p, seed, offset), K.Shard(row0, col0, ng), cuda_dev).cpu().numpy()
    want = philox.keep_mask(M, N, p, seed, offset, row0=row0, col0=col0, n_global=ng or None)
    assert got.dtype == np.uint8 and np.array_equal(got.astype(bool), want)


def test_mask_applied_by_forward_equals_dumped_mask(pkg, cuda_dev):
    """H with dropout == H without dropout * mask / (1-p), element for element."""
    K = pkg.ops.kernels
    g = torch.Generator().manual_seed(0)
    x = torch.randn((192, 128), generator=g).to(torch.bfloat16).to(cuda_dev)
    wg = (torch.randn((256, 128), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    wu = (torch.randn((256, 128), generator=g) * 0.1).to(torch.bfloat16).to(cuda_dev)
    drop = K.Dropout(0.3, 42, 5)
    h0 = K.hidden_fwd(x, wg, None, wu, None).float()
    h1 = K.hidden_fwd(x, wg, None, wu, None, drop=drop).float()
    mask = K.dropout_mask(192, 256, drop, device=cuda_dev).bool()
    assert torch.equal(h1 == 0, (~mask) | (h0 == 0))
    want = (h0 * float(philox.scale(0.3))).to(torch.bfloat16).float()
    close = (h1[mask] - want[mask]).abs() <= 2 ** -7 * want[mask].abs() + 1e-6
    assert close.all()
