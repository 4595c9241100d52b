"""ctypes loader for libbmxk.so, the C-ABI CUDA library.

The library is built in-tree by `python -m bmx_b200.build`.  There is no fallback: if it is
missing or fails to load, importing the kernels raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbmxk.so")

BMXK_OK, BMXK_ERR_INVALID, BMXK_ERR_CUDA, BMXK_ERR_DEVICE = 0, 1, 2, 3
DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2


class K2bGeom(ctypes.Structure):
    """Mirror of `bmxk_k2b_geom` (include/bmxk.h)."""

    _fields_ = [(n, c_int32) for n in
                ("h_kv", "n_q_groups", "page", "rank", "group", "n_coef_heads", "kbits", "vbits", "layout")]


class RtnGeom(ctypes.Structure):
    """Mirror of `bmxk_rtn_geom` (include/bmxk.h)."""

    _fields_ = [(n, c_int32) for n in
                ("h_kv", "n_q_groups", "page", "k_arm", "k_group", "v_group", "kbits", "vbits")]


class SpectralGeom(ctypes.Structure):
    """Mirror of `bmxk_spectral_geom` (include/bmxk.h)."""

    _fields_ = [(n, c_int32) for n in ("h_kv", "page", "group", "block_bytes", "scale_off")]


class BmxkError(RuntimeError):
    """A bmxk entry point returned a non-zero status."""

    def __init__(self, fn: str, code: int, msg: str):
        super().__init__(f"{fn} failed with status {code}: {msg}")
        self.code = code


_SIGNATURES = {
    "bmxk_version": (c_int, []),
    "bmxk_last_error": (c_char_p, []),
    "bmxk_pack_u": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "bmxk_unpack_u": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "bmxk_pack_s4": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "bmxk_unpack_s4": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p]),
    "bmxk_k2b_page_block_bytes": (c_size_t, [POINTER(K2bGeom)]),
    "bmxk_k2b_coef_block_bytes": (c_size_t, [POINTER(K2bGeom)]),
    "bmxk_k2b_append": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
                                 c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                 c_void_p]),
    "bmxk_k2b_append_coefs": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                       c_void_p]),
    "bmxk_k2b_export_stacks": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "bmxk_k2b_dequant_pages": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "bmxk_k2b_decode_workspace_bytes": (c_size_t, [POINTER(K2bGeom), c_int, c_int]),
    "bmxk_k2b_decode": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                 c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                 c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_size_t, c_void_p,
                                 c_int, c_void_p, c_int, c_void_p]),
    "bmxk_k2b_prefill": (c_int, [POINTER(K2bGeom), c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                 c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float,
                                 c_void_p, c_void_p, c_void_p]),
    "bmxk_k2b_prefill_select": (c_int, [c_int]),
    "bmxk_k2b_prefill_workspace_bytes": (c_size_t, [POINTER(K2bGeom), c_int, c_int, c_int]),
    "bmxk_k2b_prefill_split": (c_int, [POINTER(K2bGeom), c_void_p, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                       c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_float,
                                       c_void_p, c_void_p, c_int, c_void_p, c_size_t, c_void_p]),
    "bmxk_k2b_dequant_dense": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                       c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int, c_void_p]),
    "bmxk_k2b_decode_static": (c_int, [POINTER(K2bGeom), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                        c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,
                                        c_void_p, c_int, c_void_p, c_void_p, c_float, c_void_p, c_int, c_void_p]),
    "bmxk_k2b_make_v_lut": (c_int, [POINTER(c_float), POINTER(c_uint32)]),
    "bmxk_rtn_page_block_bytes": (c_size_t, [POINTER(RtnGeom)]),
    "bmxk_rtn_decode_workspace_bytes": (c_size_t, [POINTER(RtnGeom), c_int, c_int]),
    "bmxk_rtn_append": (c_int, [POINTER(RtnGeom), c_void_p, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int,
                                 c_int, c_void_p, c_void_p]),
    "bmxk_rtn_export": (c_int, [POINTER(RtnGeom), c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p]),
    "bmxk_rtn_decode": (c_int, [POINTER(RtnGeom), c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p, c_int, c_float, c_void_p, c_size_t, c_void_p, c_int, c_void_p,
                                 c_void_p]),
    "bmxk_spectral_append": (c_int, [POINTER(SpectralGeom), c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                      c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "bmxk_spectral_dequant_pages": (c_int, [POINTER(SpectralGeom), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                                             c_void_p, c_void_p, c_void_p, c_void_p]),
    "bmxk_vblock_bytes": (c_size_t, []),
    "bmxk_vblock_append": (c_int, [c_int, c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                   c_void_p, c_void_p]),
    "bmxk_vblock_export": (c_int, [c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p]),
    "bmxk_spectral_decode_workspace_bytes": (c_size_t, [POINTER(SpectralGeom), c_int, c_int]),
    "bmxk_spectral_decode": (c_int, [POINTER(SpectralGeom), c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p,
                                      c_int, c_void_p, c_void_p, c_float, c_void_p, c_size_t, c_void_p, c_int, c_void_p, c_int,
                                      c_void_p]),
    "bmxk_merge_partials": (c_int, [c_void_p, c_int, c_int, c_void_p, c_int, c_void_p]),
    "bmxk_xchg_bytes": (c_size_t, [c_int, c_int]),
    "bmxk_xchg_alloc": (c_int, [c_int, c_int, POINTER(c_void_p), c_void_p]),
    "bmxk_xchg_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "bmxk_xchg_close": (c_int, [c_void_p]),
    "bmxk_xchg_free": (c_int, [c_void_p]),
    "bmxk_xchg_merge": (c_int, [c_void_p, c_int, c_int, c_int, POINTER(c_void_p), c_int, c_int64, c_void_p, c_void_p, c_int, c_void_p]),
    "bmxk_window_append": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_int, c_int, c_int, c_int, c_void_p]),
    "bmxk_window_append_devpos": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "bmxk_gather_next_slots": (c_int, [c_void_p, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]),
    "bmxk_window_shift": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p]),
    "bmxk_step_ingest": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "bmxk_check_workspace_status": (c_int, [c_void_p, c_void_p]),
    "bmxk_k2b_decode_static_status": (c_int, [c_void_p]),
    "bmxk_selftest_bounded_wait": (c_int, [c_void_p, ctypes.c_int64, c_void_p]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library with argument types set; raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is not built; run `python -m bmx_b200.build` (needs nvcc). "
                "There is no CPU or PyTorch fallback for the bmxk kernels.")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here means header and library disagree
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def exported_symbols() -> list[str]:
    return sorted(_SIGNATURES)


def check(fn_name: str, status: int) -> None:
    if status != BMXK_OK:
        raise BmxkError(fn_name, status, lib().bmxk_last_error().decode())


def call(fn_name: str, *args) -> None:
    """Calls an int-returning entry point and raises BmxkError on a non-zero status."""
    check(fn_name, getattr(lib(), fn_name)(*args))
