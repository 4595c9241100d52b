"""Named KV-compression recipes: arm string -> (k_spec, v_spec).

Same names, parameters and parsing rules as bmx's registry (bmx: src/bmx/cache/recipes.py:13-178).
"""

from __future__ import annotations

from .specs import CacheCodecSpec


def _parse_k_r(body: str) -> tuple[int, int]:
    bits_str, rank_str = body.split("r")
    return int(bits_str), int(rank_str)


def spec_pair(arm: str, *, rank: int = 16, group: int = 64, seed: int = 0,
              pack_path: str = "") -> tuple[CacheCodecSpec, CacheCodecSpec]:
    """(k_spec, v_spec) for a named arm; raises ValueError for an unknown one."""
    if arm == "fp16":
        return CacheCodecSpec(arm="fp16"), CacheCodecSpec(arm="fp16")
    if arm == "k2b_ph":  # low-rank K @3b pre-RoPE + per-head Hadamard/Lloyd V @2b: the fused recipe
        return (CacheCodecSpec(arm="lowrank_rtn_channel", bits=3, rank=rank, group=group, seed=seed, pre_rope=True),
                CacheCodecSpec(arm="turboquant_mse_perhead", bits=2, seed=seed))
    if arm == "k2b" or arm.startswith("k2b_k"):
        bits_k, rank_k = (3, rank) if arm == "k2b" else _parse_k_r(arm[len("k2b_k"):])
        return (CacheCodecSpec(arm="lowrank_rtn_channel", bits=bits_k, rank=rank_k, group=group, seed=seed, pre_rope=True),
                CacheCodecSpec(arm="turboquant_mse", bits=2, seed=seed))
    if arm == "k2t" or arm.startswith("k2t_k"):
        bits_k, rank_k = (2, rank) if arm == "k2t" else _parse_k_r(arm[len("k2t_k"):])
        return (CacheCodecSpec(arm="lowrank_turboquant", bits=bits_k, rank=rank_k, group=group, seed=seed, pre_rope=True),
                CacheCodecSpec(arm="turboquant_mse", bits=2, seed=seed))
    if arm.startswith("k4_b"):
        if not pack_path:
            raise ValueError("k4 arms require --pack-path (a fitted spectral pack file)")
        budget_str = arm[len("k4_b"):]
        dec_quant = "fp32"
        if budget_str.endswith("_dec8tl"):
            dec_quant, budget_str = "int8_tl", budget_str[: -len("_dec8tl")]
        elif "_dec8t" in budget_str:
            budget_str, _, t_str = budget_str.partition("_dec8t")
            dec_quant = f"int8_t{t_str}"
        elif budget_str.endswith("_dec8"):
            dec_quant, budget_str = "int8", budget_str[: -len("_dec8")]
        payload_quant = "rtn"
        if budget_str.endswith("_lq"):
            payload_quant, budget_str = "lloyd", budget_str[: -len("_lq")]
        if "_lq" in arm and payload_quant != "lloyd":
            raise ValueError(f"malformed k4 arm {arm!r}: '_lq' must sit between the budget and any '_dec8*' "
                             "suffix, e.g. 'k4_b2.5_lq_dec8tl'")
        return (CacheCodecSpec(arm="spectral", pre_rope=True, group=group, pack_path=pack_path,
                               budget=float(budget_str), dec_quant=dec_quant, payload_quant=payload_quant),
                CacheCodecSpec(arm="turboquant_mse", bits=2, seed=seed))
    if arm in ("turboquant_mse", "turboquant_prod"):
        s = CacheCodecSpec(arm=arm, bits=2, seed=seed)
        return s, s
    if arm.startswith("turboquant_mse_b") or arm.startswith("turboquant_prod_b"):
        base, _, bits_str = arm.rpartition("_b")
        s = CacheCodecSpec(arm=base, bits=int(bits_str), seed=seed)
        return s, s
    if arm.startswith("turboquant_mse_k") or arm.startswith("turboquant_prod_k"):
        base, _, body = arm.rpartition("_k")
        bk, _, bv = body.partition("v")
        return CacheCodecSpec(arm=base, bits=int(bk), seed=seed), CacheCodecSpec(arm=base, bits=int(bv), seed=seed)
    if arm == "kivi":
        return (CacheCodecSpec(arm="rtn_channel", bits=2, group=group, seed=seed),
                CacheCodecSpec(arm="rtn_token", bits=2, group=group, seed=seed))
    raise ValueError(f"unknown arm {arm!r}")
