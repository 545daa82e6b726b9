"""ctypes binding of libllsa_b200.so (the C ABI declared in include/llsa_b200.h).

The library is the only compute path: if it cannot be loaded (and cannot be
built because nvcc is absent) importing an op raises -- there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libllsa_b200.so")

F32, BF16, I32, I64 = 0, 1, 2, 3
_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.int32: I32, torch.int64: I64}


class LlsaTensor(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("dtype", C.c_int32), ("ndim", C.c_int32),
                ("shape", C.c_int64 * 4), ("stride", C.c_int64 * 4)]


class LlsaAttnArgs(C.Structure):
    _P = C.POINTER(LlsaTensor)
    _fields_ = [
        ("q", _P), ("k", _P), ("v", _P), ("pk", _P), ("pv", _P), ("pk2", _P), ("pv2", _P),
        ("indices", _P), ("p_indices", _P), ("o", _P), ("lse", _P),
        ("topk", C.c_int32), ("topk_p", C.c_int32), ("block_size", C.c_int32),
        ("token_weight", C.c_float), ("token_weight_2", C.c_float),
        ("d_o", _P), ("dq", _P), ("dk", _P), ("dv", _P), ("offsets", _P), ("flat", _P), ("delta", _P),
        ("dpk_acc", _P), ("dpv_acc", _P), ("dpk2_acc", _P), ("dpv2_acc", _P),
        ("fold_pool_bwd", C.c_int32), ("kv_weight", C.c_float), ("kv_weight_2", C.c_float),
        ("force_generic", C.c_int32), ("stage_mask", C.c_int32), ("dkv_partial", _P),
        ("fine_pds", _P), ("flat_pairs", _P), ("flat_ranges", _P), ("no_tcgen05", C.c_int32), ("wait_limit", C.c_int32), ("status", C.c_void_p),
        ("fwd_redo", _P),
    ]


EXPORTS = [
    "llsa_version", "llsa_last_error_string", "llsa_mean_pool_fwd", "llsa_mean_pool_bwd", "llsa_pool_pyramid_fwd",
    "llsa_rope_pool_pyramid_fwd", "llsa_rms_rope_pool_pyramid_fwd", "llsa_rms_norm_fwd",
    "llsa_rope_fwd", "llsa_rope_bwd", "llsa_coarse_topk", "llsa_refine_topk", "llsa_select_two_level", "llsa_transpose_scratch_bytes",
    "llsa_transpose_indices", "llsa_transpose_indices_pairs", "llsa_transpose_range_entries", "llsa_transpose_indices_noalloc", "llsa_attn_fwd", "llsa_attn_bwd",
    "llsa_attn_bwd_partial_elems", "llsa_attn_bwd_pds_elems", "llsa_status_check",
]

_lib: Optional[C.CDLL] = None
_lock = threading.Lock()


def _declare(lib: C.CDLL) -> None:
    TP = C.POINTER(LlsaTensor)
    lib.llsa_version.restype = C.c_int
    lib.llsa_last_error_string.restype = C.c_char_p
    lib.llsa_mean_pool_fwd.argtypes = [TP, TP, C.c_int, C.c_void_p]
    lib.llsa_mean_pool_bwd.argtypes = [TP, TP, C.c_int, C.c_void_p]
    lib.llsa_pool_pyramid_fwd.argtypes = [C.c_int, TP, TP, TP, C.c_int, C.c_void_p]
    lib.llsa_rope_pool_pyramid_fwd.argtypes = [C.c_int, TP, TP, C.c_int, TP, TP, TP, C.c_int, C.c_void_p]
    lib.llsa_rms_rope_pool_pyramid_fwd.argtypes = [C.c_int, TP, C.POINTER(TP), C.c_int, C.c_float, TP, C.c_int, TP, TP, TP, C.c_int, C.c_void_p]
    lib.llsa_rms_norm_fwd.argtypes = [TP, TP, C.c_float, TP, C.c_void_p]
    lib.llsa_rope_fwd.argtypes = [TP, TP, TP, C.c_void_p]
    lib.llsa_rope_bwd.argtypes = [TP, TP, TP, C.c_void_p]
    lib.llsa_coarse_topk.argtypes = [TP, TP, TP, C.c_int, C.c_void_p]
    lib.llsa_refine_topk.argtypes = [TP, TP, TP, TP, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.llsa_select_two_level.argtypes = [TP, TP, TP, TP, TP, TP, C.c_int, C.c_int, C.c_int, C.c_void_p]
    lib.llsa_transpose_range_entries.argtypes = [C.c_int64] * 4
    lib.llsa_transpose_scratch_bytes.argtypes = [C.c_int64] * 5
    lib.llsa_transpose_scratch_bytes.restype = C.c_size_t
    lib.llsa_transpose_indices.argtypes = [TP, TP, TP, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.llsa_transpose_indices_noalloc.argtypes = [TP, TP, TP, C.c_int64, C.c_void_p, C.c_void_p]
    lib.llsa_attn_bwd_partial_elems.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int32]
    lib.llsa_attn_bwd_partial_elems.restype = C.c_int64
    lib.llsa_transpose_indices_pairs.argtypes = [TP, TP, TP, TP, TP, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]
    lib.llsa_attn_bwd_pds_elems.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_int32]
    lib.llsa_attn_bwd_pds_elems.restype = C.c_int64
    lib.llsa_status_check.argtypes = [C.c_int32]
    lib.llsa_attn_fwd.argtypes = [C.POINTER(LlsaAttnArgs), C.c_void_p]
    lib.llsa_attn_bwd.argtypes = [C.POINTER(LlsaAttnArgs), C.c_void_p]
    for name in EXPORTS:
        fn = getattr(lib, name)
        if name not in ("llsa_last_error_string", "llsa_transpose_scratch_bytes", "llsa_attn_bwd_partial_elems", "llsa_attn_bwd_pds_elems"):
            fn.restype = C.c_int


def lib() -> C.CDLL:
    """The loaded shared library; builds it with nvcc first if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                from . import build as _build   # raises if nvcc is unavailable: no silent fallback
                _build.build()
            try:
                handle = C.CDLL(LIB_PATH)
            except OSError as e:   # pragma: no cover
                raise RuntimeError("llsa_b200: cannot load %s (%s); run `python -m llsa_b200.build`" % (LIB_PATH, e))
            _declare(handle)
            _lib = handle
    return _lib


def desc(t: Optional[torch.Tensor]) -> Optional[LlsaTensor]:
    if t is None:
        return None
    d = LlsaTensor()
    d.ptr = t.data_ptr()
    d.dtype = _DTYPES[t.dtype]
    d.ndim = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.stride[i] = t.stride(i)
    return d


def ref(d: Optional[LlsaTensor]):
    return C.byref(d) if d is not None else None


def ptr(d: Optional[LlsaTensor]):
    return C.pointer(d) if d is not None else C.POINTER(LlsaTensor)()


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError("llsa_b200.%s failed (code %d): %s" % (what, rc, lib().llsa_last_error_string().decode()))


def stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)
