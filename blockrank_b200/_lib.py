"""ctypes binding of libblockrank_b200.so (the C ABI in include/blockrank_b200.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised.  Build the library with ``python -m blockrank_b200.build``.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libblockrank_b200.so")

BRK_BF16, BRK_F32 = 0, 1
ALGO_AUTO, ALGO_SIMT, ALGO_TC = 0, 1, 2
ERRORS = {-1: "BRK_E_ARG", -2: "BRK_E_UNSUPPORTED", -3: "BRK_E_WORKSPACE", -4: "BRK_E_CUDA",
          -5: "BRK_E_DEVICE", -6: "BRK_E_TIMEOUT"}

EXPORTS = ("brk_version", "brk_last_error", "brk_device_check", "brk_spans_from_mask",
           "brk_attn_fwd_workspace_bytes", "brk_attn_fwd", "brk_attn_bwd_workspace_bytes", "brk_attn_bwd",
           "brk_status_poll", "brk_selftest_bounded_wait",
           "brk_doc_scores_workspace_bytes",
           "brk_doc_scores", "brk_doc_scores_static", "brk_raw_scores", "brk_rmsnorm", "brk_rope", "brk_silu_mul")


class View(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("stride_b", C.c_int64), ("stride_h", C.c_int64), ("stride_s", C.c_int64)]


class AttnParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("algo", C.c_int32), ("B", C.c_int32), ("N", C.c_int32), ("Nk", C.c_int32),
                ("D", C.c_int32), ("S", C.c_int32), ("M", C.c_int32), ("max_block_len", C.c_int32),
                ("scale", C.c_float), ("q", View), ("k", View), ("v", View), ("o", View),
                ("lse", C.c_void_p), ("blk_start", C.c_void_p), ("blk_len", C.c_void_p), ("status", C.c_void_p),
                ("max_query_len", C.c_int32)]


class AttnBwdParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("B", C.c_int32), ("N", C.c_int32), ("Nk", C.c_int32), ("D", C.c_int32),
                ("S", C.c_int32), ("M", C.c_int32), ("max_block_len", C.c_int32), ("scale", C.c_float),
                ("q", View), ("k", View), ("v", View), ("o", View), ("d_o", View), ("lse", C.c_void_p),
                ("blk_start", C.c_void_p), ("blk_len", C.c_void_p), ("dq", View), ("dk", View), ("dv", View)]


class ScoreParams(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("B", C.c_int32), ("N", C.c_int32), ("Nk", C.c_int32), ("D", C.c_int32),
                ("S", C.c_int32), ("M", C.c_int32), ("R", C.c_int32), ("scale", C.c_float),
                ("temperature", C.c_float), ("q", View), ("k", View), ("rows", C.c_void_p),
                ("blk_start", C.c_void_p), ("blk_len", C.c_void_p), ("doc_mass", C.c_void_p),
                ("logits", C.c_void_p)]


class BlockRankLibraryError(RuntimeError):
    pass


_lib = None


def lib() -> C.CDLL:
    """Load the shared library once; raise ImportError if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: the BlockRank CUDA kernels are not built. "
            "Run `python -m blockrank_b200.build` (needs nvcc); there is no CPU or PyTorch fallback.")
    L = C.CDLL(LIB_PATH)
    L.brk_version.restype = C.c_int
    L.brk_last_error.restype = C.c_char_p
    L.brk_device_check.restype = C.c_int
    L.brk_spans_from_mask.restype = C.c_int
    L.brk_spans_from_mask.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    L.brk_attn_fwd_workspace_bytes.restype = C.c_size_t
    L.brk_attn_fwd_workspace_bytes.argtypes = [C.POINTER(AttnParams)]
    L.brk_attn_fwd.restype = C.c_int
    L.brk_attn_fwd.argtypes = [C.POINTER(AttnParams), C.c_void_p, C.c_size_t, C.c_void_p]
    L.brk_attn_bwd_workspace_bytes.restype = C.c_size_t
    L.brk_attn_bwd_workspace_bytes.argtypes = [C.POINTER(AttnBwdParams)]
    L.brk_attn_bwd.restype = C.c_int
    L.brk_attn_bwd.argtypes = [C.POINTER(AttnBwdParams), C.c_void_p, C.c_size_t, C.c_void_p]
    L.brk_status_poll.restype = C.c_int
    L.brk_status_poll.argtypes = [C.c_void_p, C.c_void_p]
    L.brk_selftest_bounded_wait.restype = C.c_int
    L.brk_selftest_bounded_wait.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p]
    L.brk_doc_scores_workspace_bytes.restype = C.c_size_t
    L.brk_doc_scores_workspace_bytes.argtypes = [C.POINTER(ScoreParams)]
    L.brk_doc_scores.restype = C.c_int
    L.brk_doc_scores.argtypes = [C.POINTER(ScoreParams), C.c_void_p, C.c_size_t, C.c_void_p]
    L.brk_doc_scores_static.restype = C.c_int
    L.brk_doc_scores_static.argtypes = [C.POINTER(ScoreParams), C.c_void_p]
    L.brk_raw_scores.restype = C.c_int
    L.brk_raw_scores.argtypes = [C.POINTER(ScoreParams), C.c_void_p, C.c_void_p]
    L.brk_rmsnorm.restype = C.c_int
    L.brk_rmsnorm.argtypes = [C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32,
                              C.c_float, C.c_void_p]
    L.brk_rope.restype = C.c_int
    L.brk_rope.argtypes = [C.c_int32, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int64, C.c_int32, C.c_int32,
                           C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    L.brk_silu_mul.restype = C.c_int
    L.brk_silu_mul.argtypes = [C.c_int32, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]
    _lib = L
    return L


def check(rc: int, what: str) -> None:
    """Turn a negative status into an exception carrying the library's message."""
    if rc == 0:
        return
    msg = lib().brk_last_error().decode("utf-8", "replace")
    name = ERRORS.get(rc, str(rc))
    if rc in (-1, -2, -3):
        raise ValueError(f"{what}: {name}: {msg}")
    raise BlockRankLibraryError(f"{what}: {name}: {msg}")
