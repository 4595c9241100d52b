"""The C-ABI library loads, exports every symbol include/bmxk.h declares, and rejects bad
arguments on the host before any launch (no GPU needed for any of this)."""

import ctypes
import os
import re

import pytest

from bmx_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.lib()


def _declared():
    text = open(os.path.join(ROOT, "include", "bmxk.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bmxk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/bmxk.h but not exported"
    assert set(names) == set(_lib.exported_symbols()), "ctypes signatures and header disagree"
    assert lib.bmxk_version() >= 100


def test_argument_errors_are_reported_not_launched(lib):
    assert lib.bmxk_pack_u(None, None, 2, 64, 3, None) == _lib.BMXK_ERR_INVALID
    assert b"bits" in lib.bmxk_last_error()
    assert lib.bmxk_pack_s4(None, None, 2, 63, 3, None) == _lib.BMXK_ERR_INVALID
    assert lib.bmxk_pack_u(None, None, 0, 64, 2, None) == _lib.BMXK_OK  # empty input: nothing to do
    g = _lib.K2bGeom(8, 4, 100, 32, 64, 8, 3, 2)
    assert lib.bmxk_k2b_append(ctypes.byref(g), None, None, 0, 0, 0, 128, None, None, None, None, 1, 1, None, None,
                               None) == _lib.BMXK_ERR_INVALID
    assert b"page" in lib.bmxk_last_error()
    g = _lib.K2bGeom(8, 4, 128, 32, 64, 8, 3, 2)
    assert lib.bmxk_k2b_page_block_bytes(ctypes.byref(g)) == 128 * 64 + 2 * 128 * 2 + 128 * 32 + 128 * 2
    assert lib.bmxk_k2b_coef_block_bytes(ctypes.byref(g)) == 128 * 32 * 2
    with pytest.raises(_lib.BmxkError):
        _lib.call("bmxk_merge_partials", None, 0, 0, None, 0, None)
    # fused spectral decode: 64-token pages and inconsistent block sizes are refused before any launch
    sg = _lib.SpectralGeom(8, 64, 64, 7424, 6400)
    args = [4, None, None, None, None, None, None, 0, None, 1, 1, None, None, 0, None, None, None, 0, None, None, 0.1, None, 0, None, 0,
            None, 3, None]
    assert lib.bmxk_spectral_decode(ctypes.byref(sg), *args) == _lib.BMXK_ERR_INVALID
    assert b"page" in lib.bmxk_last_error()
    sg = _lib.SpectralGeom(8, 128, 64, 7424, 7000)
    assert lib.bmxk_spectral_decode(ctypes.byref(sg), *args) == _lib.BMXK_ERR_INVALID
    assert b"block_bytes" in lib.bmxk_last_error()
    assert lib.bmxk_vblock_bytes() == 128 * 32 + 128 * 2
    assert lib.bmxk_vblock_append(0, None, 0, 0, 0, 0, None, None, None, 1, 1, None, None) == _lib.BMXK_ERR_INVALID


def test_value_table_is_exact_to_1e6(lib):
    import struct

    import numpy as np

    from bmx_b200.kernels import GAUSSIAN_CODEBOOK, make_v_lut

    lo, hi, a, b = make_v_lut(GAUSSIAN_CODEBOOK[2])
    alpha = struct.unpack("<f", struct.pack("<I", a))[0]
    beta = struct.unpack("<f", struct.pack("<I", b))[0]
    for i, level in enumerate(GAUSSIAN_CODEBOOK[2]):
        bits = ((hi >> (8 * i)) & 0xFF) << 8 | ((lo >> (8 * i)) & 0xFF)
        h = float(np.frombuffer(struct.pack("<H", bits), dtype=np.float16)[0])
        assert abs(alpha + beta * h - level) < 2e-6
    assert abs(alpha) < 0.02
