"""ctypes binding of libgmlp.so (C ABI declared in include/gmlp.h).

There is no fallback: if the library is missing or a call fails, the caller gets
an exception that names the problem. Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

LIB_PATH = Path(__file__).resolve().parent / "libgmlp.so"

GMLP_BF16, GMLP_FP16, GMLP_F32 = 0, 1, 2

# gmlp_act_t by the names the reference's module accepts (gated_mlp.py:27-37)
ACT_CODES = {"silu": 0, "swish": 0, "no_act": 1, "relu": 2, "gelu": 3, "sigmoid": 4, "tanh": 5, "leaky_relu": 6}

# Every symbol include/gmlp.h declares; tests check that the library exports all of them.
EXPORTS = (
    "gmlp_hidden_fwd", "gmlp_hidden_fwd_scaled", "gmlp_rms_rowscale", "gmlp_rms_bwd", "gmlp_decode_fwd_scaled",
    "gmlp_decode_fwd_fused",
    "gmlp_quantize_rows_e4m3", "gmlp_decode_fwd_fp8",
    "gmlp_down_fwd", "gmlp_mlp_fwd", "gmlp_mlp_bwd", "gmlp_bwd_dhidden", "gmlp_bwd_dact", "gmlp_bwd_dx",
    "gmlp_bwd_dw_gate_up", "gmlp_bwd_dw_down", "gmlp_bias_grad_scratch_bytes", "gmlp_bwd_dw_gate_up_bias",
    "gmlp_bwd_dw_down_bias", "gmlp_colsum_scratch_bytes", "gmlp_colsum", "gmlp_colsum_static",
    "gmlp_dropout_mask", "gmlp_gemm", "gmlp_decode_scratch_bytes", "gmlp_decode_fwd", "gmlp_set_cta_pair_mode", "gmlp_set_raster_group", "gmlp_set_sm_limit",
    "gmlp_peer_region_bytes", "gmlp_set_peer_two_shot_bytes", "gmlp_peer_alloc", "gmlp_peer_open", "gmlp_peer_close", "gmlp_peer_free",
    "gmlp_peer_allreduce", "gmlp_down_fwd_push", "gmlp_bwd_dx_push", "gmlp_peer_reduce_gather", "gmlp_status_read", "gmlp_last_error", "gmlp_version",
)


class GmlpError(RuntimeError):
    pass


class Problem(C.Structure):
    """Mirror of gmlp_problem_t."""

    _fields_ = [
        ("M", C.c_int64), ("K", C.c_int64), ("N", C.c_int64),
        ("dtype", C.c_int32), ("dropout_p", C.c_float),
        ("seed", C.c_uint64), ("offset", C.c_uint64),
        ("row0_global", C.c_int64), ("col0_global", C.c_int64), ("N_global", C.c_int64),
        ("act", C.c_int32), ("tuning", C.c_uint32),
    ]


_lib = None


def _declare(lib: C.CDLL) -> None:
    vp, i32, i64, u8p = C.c_void_p, C.c_int32, C.c_int64, C.c_void_p
    pp = C.POINTER(Problem)
    lib.gmlp_hidden_fwd.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_hidden_fwd_scaled.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_rms_rowscale.argtypes = [i64, i64, i32, vp, i64, C.c_float, vp, vp, vp]
    lib.gmlp_rms_bwd.argtypes = [i64, i64, i32, vp, vp, vp, vp, vp]
    lib.gmlp_decode_fwd_scaled.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, C.c_size_t, vp]
    lib.gmlp_decode_fwd_fused.argtypes = lib.gmlp_decode_fwd_scaled.argtypes
    lib.gmlp_quantize_rows_e4m3.argtypes = [i64, i64, i32, vp, i64, vp, vp, vp]
    lib.gmlp_decode_fwd_fp8.argtypes = [pp] + [vp] * 18 + [C.c_size_t, vp]
    lib.gmlp_down_fwd.argtypes = [pp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_mlp_fwd.argtypes = [pp] + [vp] * 13
    lib.gmlp_mlp_bwd.argtypes = [pp] + [vp] * 18 + [C.c_size_t, vp]
    lib.gmlp_bwd_dhidden.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_bwd_dact.argtypes = [pp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_bwd_dx.argtypes = [pp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_bwd_dw_gate_up.argtypes = [pp, vp, vp, vp, vp, vp, vp]
    lib.gmlp_bwd_dw_down.argtypes = [pp, vp, vp, vp, vp]
    lib.gmlp_bias_grad_scratch_bytes.argtypes = [pp]
    lib.gmlp_bias_grad_scratch_bytes.restype = C.c_size_t
    lib.gmlp_bwd_dw_gate_up_bias.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, C.c_size_t, vp]
    lib.gmlp_bwd_dw_down_bias.argtypes = [pp, vp, vp, vp, vp, vp, C.c_size_t, vp]
    lib.gmlp_colsum_scratch_bytes.argtypes = [i64, i64]
    lib.gmlp_colsum_scratch_bytes.restype = C.c_size_t
    lib.gmlp_colsum.argtypes = [i64, i64, i32, vp, i64, vp, C.c_size_t, vp, vp]
    lib.gmlp_colsum_static.argtypes = [i64, i64, i32, vp, i64, vp, vp]
    lib.gmlp_dropout_mask.argtypes = [pp, u8p, vp]
    lib.gmlp_gemm.argtypes = [i32, i32, i32, i64, i64, i64, vp, i64, vp, i64, vp, i64, vp, vp]
    lib.gmlp_decode_scratch_bytes.argtypes = [pp]
    lib.gmlp_decode_scratch_bytes.restype = C.c_size_t
    lib.gmlp_decode_fwd.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, C.c_size_t, vp]
    lib.gmlp_set_cta_pair_mode.argtypes = [i32]
    lib.gmlp_set_raster_group.argtypes = [i32]
    lib.gmlp_set_sm_limit.argtypes = [i32]
    lib.gmlp_set_peer_two_shot_bytes.argtypes = [C.c_longlong]
    lib.gmlp_set_peer_two_shot_bytes.restype = C.c_longlong
    lib.gmlp_peer_region_bytes.argtypes = [i64, i32]
    lib.gmlp_peer_region_bytes.restype = C.c_size_t
    lib.gmlp_peer_alloc.argtypes = [C.c_size_t, C.POINTER(vp), vp]
    lib.gmlp_peer_open.argtypes = [vp, C.POINTER(vp)]
    lib.gmlp_peer_close.argtypes = [vp]
    lib.gmlp_peer_free.argtypes = [vp]
    lib.gmlp_peer_allreduce.argtypes = [i32, i64, i64, vp, C.POINTER(vp), i32, i32, vp, i32, vp]
    lib.gmlp_down_fwd_push.argtypes = [pp, vp, vp, vp, vp, vp, i64, C.POINTER(vp), i32, i32, vp]
    lib.gmlp_peer_reduce_gather.argtypes = [i32, i64, i64, vp, C.POINTER(vp), i32, i32, vp]
    lib.gmlp_bwd_dx_push.argtypes = [pp, vp, vp, vp, vp, vp, i64, C.POINTER(vp), i32, i32, vp]
    lib.gmlp_status_read.argtypes = [C.POINTER(C.c_int)]
    lib.gmlp_last_error.restype = C.c_char_p
    lib.gmlp_version.restype = C.c_int
    for name in EXPORTS:
        getattr(lib, name)  # AttributeError here means the library and the header disagree


def load() -> C.CDLL:
    """Load libgmlp.so from the package directory (built in-tree by build.py)."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise GmlpError(
                f"{LIB_PATH} is missing: run `python __graft_entry__.py` (or the package's "
                "build.build()) to compile the sm_100a kernels. There is no CPU or Triton fallback."
            )
        lib = C.CDLL(str(LIB_PATH))
        _declare(lib)
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        raise GmlpError(f"libgmlp error {rc}: {load().gmlp_last_error().decode()}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.bfloat16:
        return GMLP_BF16
    if dt == torch.float16:
        return GMLP_FP16
    if dt == torch.float32:
        return GMLP_F32   # fp32 matrices, tf32 products: the compatibility path
    raise NotImplementedError(
        f"libgmlp computes in bfloat16, float16 or float32 (tf32 products); got {dt}. "
        "Convert the module and its input with .to(torch.bfloat16), .to(torch.float16) or .to(torch.float32)."
    )


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise GmlpError("libgmlp has no CPU path: every tensor must live on a CUDA (sm_100a) device")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise GmlpError(f"tensors on different devices: {dev} and {t.device}")
    return dev


_scratch_epoch = 0


def scratch_epoch() -> int:
    """Counts the non-zero status words read so far. Scratch that kernels keep zeroed between
    calls (the decode counters) may be dirty after a kernel gave up a wait; holders of such
    scratch allocate afresh when the epoch has moved."""
    return _scratch_epoch


def status_read(device: torch.device | None = None) -> int:
    """Synchronise `device` and return (and clear) its kernel status word."""
    global _scratch_epoch
    v = C.c_int(0)
    with torch.cuda.device(device):
        check(load().gmlp_status_read(C.byref(v)))
    if v.value != 0:
        _scratch_epoch += 1
    return v.value


def tune_word(pair_mode: int = 0, raster_group: int = 0, sm_limit: int = 0, ordinary_launch: bool = False,
              narrow_tiles: bool = False) -> int:
    """gmlp_problem_t.tuning for one call (the GMLP_TUNE_* fields of include/gmlp.h); 0 fields = defaults.
    ordinary_launch: decode calls only, see GMLP_TUNE_ORDINARY_LAUNCH; narrow_tiles: GMLP_TUNE_NARROW_TILES."""
    if not (0 <= pair_mode <= 2 and 0 <= raster_group <= 4095 and 0 <= sm_limit <= 4095):
        raise ValueError("pair_mode in 0..2, raster_group and sm_limit in 0..4095")
    return (pair_mode & 3) | ((raster_group & 0xFFF) << 2) | ((sm_limit & 0xFFF) << 14) | \
        ((1 << 26) if ordinary_launch else 0) | ((1 << 27) if narrow_tiles else 0)


def set_cta_pair_mode(mode: int) -> int:
    """Process-wide default: 0 = per problem, 1 = single-CTA kernel only, 2 = CTA-pair kernel only; returns the
    previous mode. A call that carries its own tune_word() is not affected."""
    return load().gmlp_set_cta_pair_mode(int(mode))


def set_raster_group(row_tiles: int) -> int:
    """Row tiles per raster group of the persistent tile order (0 = default); returns the previous value."""
    return load().gmlp_set_raster_group(int(row_tiles))


def set_sm_limit(sms: int) -> int:
    """SMs the persistent GEMM grids may occupy (0 = all); returns the previous value."""
    return load().gmlp_set_sm_limit(int(sms))
