"""ctypes front end of oracle/cpu_ref.c, the pinned-order C restatement of the k2b page quantizer.
Test infrastructure only.  Build with `make -C oracle` (done by __graft_entry__.build())."""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "libcpu_ref.so")
_lib = None


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB):
            subprocess.run(["make", "-C", _HERE, "-s"], check=True)
        _lib = ctypes.CDLL(_LIB)
    return _lib


def k2b_quant_page(M, Vv, basis, signs, codebook, *, h_kv, page, rank, group, n_coef_heads, kbits=3):
    """One page (page, C) of keys M and values Vv -> dict with bmx's stacked-tensor fields:
    us (n_coef_heads, page, rank) fp16, res_Q_int (C, page) int8, res_scale (C, page/group) fp16,
    v_idx (page, C) uint8, v_norm (page, h_kv) fp16."""
    C = h_kv * 128
    M = np.ascontiguousarray(M, np.float32)
    Vv = np.ascontiguousarray(Vv, np.float32)
    basis = np.ascontiguousarray(basis, np.float32)
    signs = np.ascontiguousarray(signs, np.float32)
    cb = np.ascontiguousarray(codebook, np.float32)
    assert M.shape == (page, C) == Vv.shape and basis.shape == (C, rank)
    out = {"us": np.zeros((n_coef_heads, page, rank), np.uint16), "res_Q_int": np.zeros((C, page), np.int8),
           "res_scale": np.zeros((C, page // group), np.uint16), "v_idx": np.zeros((page, C), np.uint8),
           "v_norm": np.zeros((page, h_kv), np.uint16)}
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)  # noqa: E731
    _load().k2b_quant_page_ref(p(M), p(Vv), p(basis), p(signs), p(cb), h_kv, page, rank, group, n_coef_heads, kbits,
                               p(out["us"]), p(out["res_Q_int"]), p(out["res_scale"]), p(out["v_idx"]), p(out["v_norm"]))
    for k in ("us", "res_scale", "v_norm"):
        out[k] = out[k].view(np.float16)
    return out
