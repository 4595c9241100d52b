"""Recipe registry and spec dataclass keep bmx's names, defaults and parsing rules
(bmx: src/bmx/cache/recipes.py, src/bmx/cache/specs.py, tests/test_recipes.py)."""

import dataclasses

import pytest

from bmx_b200.recipes import spec_pair
from bmx_b200.specs import CacheCodecSpec


def test_spec_defaults():
    s = CacheCodecSpec()
    assert dataclasses.asdict(s) == dict(arm="fp16", bits=3, rank=0, group=64, seed=0, pre_rope=False, pack_path="",
                                          budget=0.0, dec_quant="fp32", payload_quant="rtn")


def test_k2b_family():
    k, v = spec_pair("k2b_ph")
    assert (k.arm, k.bits, k.rank, k.group, k.pre_rope) == ("lowrank_rtn_channel", 3, 16, 64, True)
    assert (v.arm, v.bits) == ("turboquant_mse_perhead", 2)
    k, v = spec_pair("k2b_k2r8")
    assert (k.bits, k.rank, v.arm) == (2, 8, "turboquant_mse")
    k, v = spec_pair("k2b", rank=32, group=32, seed=3)
    assert (k.rank, k.group, k.seed, v.seed) == (32, 32, 3, 3)
    k, _ = spec_pair("k2t_k3r4")
    assert (k.arm, k.bits, k.rank) == ("lowrank_turboquant", 3, 4)


def test_k4_suffix_order_and_errors():
    with pytest.raises(ValueError):
        spec_pair("k4_b2.5")
    k, v = spec_pair("k4_b2.5_lq_dec8tl", pack_path="p")
    assert (k.arm, k.budget, k.dec_quant, k.payload_quant, k.pre_rope) == ("spectral", 2.5, "int8_tl", "lloyd", True)
    assert spec_pair("k4_b3_dec8t5", pack_path="p")[0].dec_quant == "int8_t5"
    assert spec_pair("k4_b3_dec8", pack_path="p")[0].dec_quant == "int8"
    with pytest.raises(ValueError):
        spec_pair("k4_b2.5_dec8tl_lq", pack_path="p")


def test_turboquant_kivi_and_unknown():
    k, v = spec_pair("turboquant_mse_b3")
    assert k is v and k.bits == 3
    k, v = spec_pair("turboquant_mse_k3v2")
    assert (k.bits, v.bits) == (3, 2)
    k, v = spec_pair("kivi")
    assert (k.arm, v.arm, k.bits) == ("rtn_channel", "rtn_token", 2)
    assert spec_pair("fp16")[0].arm == "fp16"
    with pytest.raises(ValueError):
        spec_pair("nope")
