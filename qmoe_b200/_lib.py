"""ctypes loader of ``libqmoe_sub1.so`` (C ABI in include/qmoe_sub1.h).

The library is the product: there is no Python or CPU fallback behind these calls.  If it is missing
or older than its sources it is rebuilt with nvcc; a failed rebuild is raised to the caller, also
when an older library exists (``QMOE_NO_BUILD=1`` loads the existing one without looking).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

from . import build as _build

OK = 0
ERR_INVALID_ARG = -1
ERR_CUDA = -2
ERR_UNSUPPORTED = -3
ERR_STREAM = -4
ERR_TIMEOUT = -5

FLAG_ACCUMULATE = 1
FLAG_RELU = 2

DICT_COUNT = 65536
TRIE_ROOT = 65536
MAX_WIDTH = 8192


class QmoeError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"qmoe status {status}: {message}")
        self.status = status


class MatrixDesc(ctypes.Structure):
    """Mirror of ``qmoe_matrix_desc``."""

    _fields_ = [
        ("code_base", ctypes.c_int64),
        ("n_codes", ctypes.c_int64),
        ("rowoff_base", ctypes.c_int64),
        ("minmax_base", ctypes.c_int64),
        ("height", ctypes.c_int32),
        ("width", ctypes.c_int32),
    ]


class InterleavedStore(ctypes.Structure):
    """Mirror of ``qmoe_interleaved_store``."""

    _fields_ = [("codes", ctypes.c_void_p), ("blk_base", ctypes.c_void_p), ("table", ctypes.c_void_p),
                ("dec", ctypes.c_void_p), ("rows", ctypes.c_void_p)]


_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_int64
_U64 = ctypes.c_uint64

# name -> (restype, argtypes); every symbol include/qmoe_sub1.h declares.
SIGNATURES = {
    "qmoe_last_error": (ctypes.c_char_p, []),
    "qmoe_version": (_I, []),
    "qmoe_sub1_build_dictionary": (_I, [_P, _P]),
    "qmoe_sub1_matvec": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _P]),
    "qmoe_sub1_matvec_noalloc": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _P]),
    "qmoe_sub1_matmul": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _L, _I, _L, _L, _I, _I, _P]),
    "qmoe_sub1_decode": (_I, [_P, _P, _P, _P, _P, _I, _I, _L, _I, _P]),
    "qmoe_sub1_pack_prepare": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "qmoe_sub1_pack_emit": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "qmoe_sub1_pack_u8_count": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "qmoe_sub1_pack_u8_gather": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "qmoe_synth_ternary": (_I, [_P, _L, _U64, _U64, ctypes.c_float, _I, _P]),
    "qmoe_moe_route": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "qmoe_moe_rank": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_keep": (_I, [_P, _P, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_scan": (_I, [_P, _P, _I, _I, _P]),
    "qmoe_moe_permute": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _L, _L, _I, _P]),
    "qmoe_moe_unpermute": (_I, [_P, _P, _P, _I, _I, _L, _L, _I, _P]),
    "qmoe_moe_work_bytes": (_L, [_I, _I, _I, _I]),
    "qmoe_moe_set_tile_min_tokens": (_I, [_I]),
    "qmoe_moe_set_items_per_matrix": (_I, [_I, _I]),
    "qmoe_moe_set_fused_phases": (_I, [_I]),
    "qmoe_moe_work_summary": (_I, [_P, _I, _I, _P, _I, _P]),
    "qmoe_moe_grouped_ffn": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_grouped_ffn_interleaved": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_grouped_ffn_rows": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _L, _P, _P, _P, _L, _P, _P, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_ep_dispatch": (_I, [_P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_plan": (_I, [_P, _L, _I, _P, _I, _I, _P, _P, _P, _I, _P]),
    "qmoe_moe_ep_dispatch_peer": (_I, [_P, _P, _L, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_plan_peer": (_I, [_P, _L, _I, _I, _I, _P, _P, _P, _P, _I, _L, _P, _I, _P]),
    "qmoe_moe_grouped_ffn_scatter": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _L, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "qmoe_moe_peer_barrier": (_I, [_P, _I, _I, _I, _L, _P, _I, _P]),
    "qmoe_moe_interleave_count": (_I, [_P, _P, _P, _I, _P, _I, _P]),
    "qmoe_moe_interleave_emit": (_I, [_P, _P, _P, _I, _P, _P, _P, _I, _P]),
    "qmoe_moe_interleave_count_rows": (_I, [_P, _P, _P, _I, _P, _P, _I, _P]),
    "qmoe_moe_interleave_emit_rows": (_I, [_P, _P, _P, _I, _P, _P, _P, _P, _I, _P]),
    "qmoe_moe_combine_add": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "qmoe_moe_route_small": (_I, [_P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _I, _P]),
    "qmoe_rms_norm": (_I, [_P, _P, _P, _I, _I, ctypes.c_float, _I, _P]),
    "qmoe_gemv": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, ctypes.c_float, _I, _I, _P]),
    "qmoe_decode_attention": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "qmoe_decode_attention_ex": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, ctypes.c_float, _P, _P, _I, _P]),
    "qmoe_sub1_code_histogram": (_I, [_P, _L, _P, _I, _P]),
    "qmoe_sub1_remap_tables": (_I, [_P, _P, _P, _P, _I, _P]),
    "qmoe_moe_combine": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _P]),
    "qmoe_launch_count": (_L, []),
    "qmoe_profile_enable": (_I, [_I]),
    "qmoe_profile_read": (_I, [_P, _P, _P]),
    "qmoe_sub1_release": (_I, [_I]),
    "qmoe_sub1_forget": (_I, [_P, _I]),
    "qmoe_moe_tile_timeouts": (_I, [_I, _I, _P]),
    "qmoe_moe_set_tile_wait_limit": (_I, [ctypes.c_uint32]),
}

_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load (building first if needed) the C-ABI library and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = _build.LIB_PATH
    if os.environ.get("QMOE_NO_BUILD") != "1" and _build.is_stale():
        # A failed rebuild is an error even when an older library exists: running a stale binary
        # after a source edit would report results of code that is no longer there.  Set
        # QMOE_NO_BUILD=1 to load whatever is built (boxes without nvcc).
        path = _build.build()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m qmoe_b200.build` (needs nvcc). "
            "There is no CPU fallback for the sub1 kernels.")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        msg = load().qmoe_last_error()
        raise QmoeError(int(status), msg.decode("utf-8", "replace") if msg else "")
