"""The C-ABI library builds, loads without a GPU, and exports exactly what include/gmlp.h declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "gmlp.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(gmlp_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    for must in ("gmlp_hidden_fwd", "gmlp_down_fwd", "gmlp_bwd_dhidden", "gmlp_bwd_dx", "gmlp_bwd_dw_gate_up",
                 "gmlp_bwd_dw_down", "gmlp_colsum", "gmlp_dropout_mask", "gmlp_last_error"):
        assert must in syms


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(str(pkg._lib.LIB_PATH))
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in gmlp.h but not exported"
    assert sorted(pkg._lib.EXPORTS) == declared_symbols(), "python binding and header disagree"


def test_version_and_error_string_need_no_gpu(pkg):
    lib = pkg._lib.load()
    assert lib.gmlp_version() >= 200   # 200: gmlp_problem_t.reserved became the per-call tuning word
    assert isinstance(lib.gmlp_last_error(), bytes)


def test_argument_checks_run_before_any_device_call(pkg):
    """Bad descriptors are rejected on the host with a status code and a message (no GPU needed)."""
    L = pkg._lib
    lib = L.load()
    ok = dict(M=4, K=64, N=64, dtype=0, dropout_p=0.0, seed=0, offset=0, row0_global=0, col0_global=0, N_global=0,
              act=0, tuning=0)

    def rc(**kw):
        p = L.Problem(**{**ok, **kw})
        return lib.gmlp_down_fwd(ctypes.byref(p), 16, 16, None, None, 16, None)

    assert rc(M=0) == -1 and b"positive" in lib.gmlp_last_error()
    assert rc(K=60) == -1
    assert rc(dtype=7) == -3
    assert rc(dropout_p=1.0) == -6
    assert rc(act=9) == -6
    p = L.Problem(**ok)
    assert lib.gmlp_down_fwd(ctypes.byref(p), None, 16, None, None, 16, None) == -6   # NULL h
    assert lib.gmlp_down_fwd(ctypes.byref(p), 8, 16, None, None, 16, None) == -2      # misaligned h
    assert lib.gmlp_hidden_fwd(ctypes.byref(p), 16, 16, None, 16, None, 16, 16, None, None) == -6  # g without u
    assert lib.gmlp_colsum(4, 12, 0, 16, 16, 16, 1 << 20, 16, None) == -1
    assert lib.gmlp_colsum(4, 16, 0, 16, 16, 16, 0, 16, None) == -7
    assert lib.gmlp_colsum_scratch_bytes(16384, 8192) >= 8192 * 4


def test_pushing_down_projection_checks_its_arguments_on_the_host(pkg):
    """gmlp_down_fwd_push / gmlp_peer_reduce_gather reject what they cannot do before any device call."""
    L = pkg._lib
    lib = L.load()
    ok = dict(M=256, K=64, N=64, dtype=0, dropout_p=0.0, seed=0, offset=0, row0_global=0, col0_global=0, N_global=0,
              act=0, tuning=0)
    regions = (ctypes.c_void_p * 2)(4096, 8192)

    def rc(world=2, rank=0, max_elems=256 * 64, regs=regions, **kw):
        p = L.Problem(**{**ok, **kw})
        return lib.gmlp_down_fwd_push(ctypes.byref(p), 16, 16, None, None, 16, max_elems, regs, rank, world, None)

    assert rc(world=1) == -6 and b"world" in lib.gmlp_last_error()
    assert rc(rank=2) == -6
    assert rc(dtype=2) == -3                           # float32 has no pushing epilogue
    assert rc(M=96) == -1 and b"32 * world" in lib.gmlp_last_error()
    assert rc(max_elems=1024) == -1 and b"capacity" in lib.gmlp_last_error()
    assert rc(regs=None) == -6
    assert lib.gmlp_peer_reduce_gather(0, 100, 1 << 20, 16, regions, 0, 2, None) == -1   # n not a multiple of 8 * world
    assert lib.gmlp_peer_reduce_gather(0, 1 << 21, 1 << 20, 16, regions, 0, 2, None) == -1  # above the capacity

