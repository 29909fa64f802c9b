"""Pins the CPU restatement of the dropout-mask generator (oracle/philox.py)."""
import numpy as np

from oracle import philox


def _kat(counter, key):
    r = philox.philox4x32_10(*[np.array([c], dtype=np.uint32) for c in counter], key[0], key[1])
    return [int(v[0]) for v in r]


def test_philox4x32_10_known_answers():
    # Known-answer vectors published with the Philox reference implementation (Random123 kat_vectors).
    assert _kat([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert _kat([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert _kat([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]) == [
        0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_threshold_and_scale():
    assert philox.threshold(0.0) == 0
    assert philox.threshold(0.5) == 2 ** 15
    assert philox.threshold(0.1) == int(float(np.float32(0.1)) * 2 ** 16) == 6553
    assert philox.threshold(0.99999) == 65535
    assert philox.scale(0.5) == np.float32(2.0)


def test_mask_rate_and_determinism():
    m1 = philox.keep_mask(256, 512, 0.1, seed=0x5EED, offset=0)
    m2 = philox.keep_mask(256, 512, 0.1, seed=0x5EED, offset=0)
    m3 = philox.keep_mask(256, 512, 0.1, seed=0x5EED, offset=1)
    assert (m1 == m2).all() and (m1 != m3).any()
    assert abs(m1.mean() - 0.9) < 5e-3
    assert philox.keep_mask(4, 8, 0.0, 1, 1).all()


def test_mask_is_invariant_to_sharding():
    full = philox.keep_mask(96, 256, 0.25, seed=3, offset=9)
    # token shard: rows 32..63
    tok = philox.keep_mask(32, 256, 0.25, seed=3, offset=9, row0=32)
    assert (tok == full[32:64]).all()
    # tensor-parallel shard: columns 128..255 of a 256-wide hidden state
    tp = philox.keep_mask(96, 128, 0.25, seed=3, offset=9, col0=128, n_global=256)
    assert (tp == full[:, 128:]).all()


def test_lane_order_within_one_generator_call():
    """Element e uses 16-bit half (e & 1) of word (e & 7) >> 1 of the call with counter e >> 3."""
    seed, offset, n = 0x1234_5678_9ABC, 3, 64
    m = philox.keep_mask(1, n, 0.5, seed, offset)
    for e in (0, 1, 6, 7, 8, 13, 63):
        w = philox.philox4x32_10(np.uint32(e >> 3), np.uint32(0), np.uint32(offset), np.uint32(0),
                                 seed & 0xFFFFFFFF, seed >> 32)
        word = int(w[(e & 7) >> 1])
        u16 = (word >> 16) if (e & 1) else (word & 0xFFFF)
        assert m[0, e] == (u16 >= 2 ** 15)


def test_mask_index_beyond_32_bits():
    # element index e = row * N crosses 2**35 here: the counter's second word must be used
    a = philox.keep_mask(2, 1024, 0.5, seed=1, offset=0, row0=(1 << 25), n_global=1024)
    b = philox.keep_mask(2, 1024, 0.5, seed=1, offset=0, row0=(1 << 25) + (1 << 23), n_global=1024)
    assert (a != b).any()
