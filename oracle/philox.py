"""CPU restatement (numpy) of the dropout-mask contract. TEST INFRASTRUCTURE ONLY.

The reference applies torch's nn.Dropout (src/triton_gated_mlp/gated_mlp.py:90,96),
whose mask depends on torch's generator and, on CUDA, on launch geometry, so it
cannot be reproduced by another kernel. The engine therefore defines its own
counter-based mask; this file is its CPU twin and the two are compared bit for
bit on the GPU box.

Generator: Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as
1, 2, 3", SC'11), restated from the published algorithm and pinned against the
paper's known-answer vectors in tests/test_oracle_philox.py.

Contract, for hidden element (row, col) of the un-sharded H[M, N_global]:
    e        = row * N_global + col
    r[0:4]   = philox4x32_10(counter = (lo32(e >> 3), hi32(e >> 3), lo32(offset), hi32(offset)),
                             key     = (lo32(seed), hi32(seed)))
    u16      = 16-bit half number (e & 1) (0 = low half) of word r[(e & 7) >> 1]
    keep     = u16 >= floor(p * 2**16)
    scale    = float32(1) / (float32(1) - float32(p))
One generator call serves 8 consecutive elements, sixteen random bits each, so the
drop probability is honoured to within 2**-16.
"""
from __future__ import annotations

import numpy as np

M0 = np.uint64(0xD2511F53)
M1 = np.uint64(0xCD9E8D57)
W0 = 0x9E3779B9
W1 = 0xBB67AE85
MASK32 = np.uint64(0xFFFFFFFF)


def philox4x32_10(c0, c1, c2, c3, k0: int, k1: int):
    """Vectorised Philox4x32-10. c0..c3: uint32 arrays (same shape); k0, k1: python ints."""
    c0 = np.asarray(c0, dtype=np.uint64)
    c1 = np.asarray(c1, dtype=np.uint64)
    c2 = np.asarray(c2, dtype=np.uint64)
    c3 = np.asarray(c3, dtype=np.uint64)
    k0 &= 0xFFFFFFFF
    k1 &= 0xFFFFFFFF
    for _ in range(10):
        p0 = M0 * c0          # 32x32 -> 64-bit products (inputs < 2**32, no overflow in uint64)
        p1 = M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & MASK32
        hi1, lo1 = p1 >> np.uint64(32), p1 & MASK32
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + W0) & 0xFFFFFFFF
        k1 = (k1 + W1) & 0xFFFFFFFF
    return (c0.astype(np.uint32), c1.astype(np.uint32), c2.astype(np.uint32), c3.astype(np.uint32))


def threshold(p: float) -> int:
    """floor(p * 2**16) with p first rounded to float32 (the C ABI carries p as a float)."""
    t = float(np.float32(p)) * 65536.0
    return int(min(t, 65535.0))


def scale(p: float) -> np.float32:
    return np.float32(1.0) / (np.float32(1.0) - np.float32(p))


def keep_mask(rows: int, cols: int, p: float, seed: int, offset: int, *, row0: int = 0, col0: int = 0,
              n_global: int | None = None) -> np.ndarray:
    """Boolean keep-mask [rows, cols] for local rows/cols placed at (row0, col0) of the global H."""
    n_global = cols if n_global is None or n_global == 0 else n_global
    if p <= 0.0:
        return np.ones((rows, cols), dtype=bool)
    assert n_global % 8 == 0 and col0 % 8 == 0 and cols % 8 == 0
    r = (np.arange(rows, dtype=np.uint64) + np.uint64(row0))[:, None]
    q = (np.arange(cols // 8, dtype=np.uint64) * np.uint64(8) + np.uint64(col0))[None, :]
    e8 = (r * np.uint64(n_global) + q) >> np.uint64(3)
    w = philox4x32_10(e8 & MASK32, e8 >> np.uint64(32), np.uint64(offset & 0xFFFFFFFF),
                      np.uint64((offset >> 32) & 0xFFFFFFFF), seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    words = np.stack(w, axis=-1)                                   # [rows, cols/8, 4]
    halves = np.stack([words & np.uint32(0xFFFF), words >> np.uint32(16)], axis=-1)  # [..., 4, 2]: low half first
    return halves.reshape(rows, cols) >= np.uint32(threshold(p))
