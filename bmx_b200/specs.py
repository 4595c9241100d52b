"""Codec specification for one side (K or V) of the KV cache.

Same dataclass, field names and defaults as bmx's (bmx: src/bmx/cache/specs.py:12-91), so that
recipes and caches built for bmx construct unchanged.
"""

from __future__ import annotations

import dataclasses


@dataclasses.dataclass
class CacheCodecSpec:
    """arm: codec name ("fp16" = no-op); bits: code width; rank: low-rank components of
    `lowrank_rtn_channel`; group: RTN group size; seed: rotation seed; pre_rope: quantize keys before
    RoPE and rotate at read; pack_path / budget / dec_quant / payload_quant: spectral (K4) arm only."""

    arm: str = "fp16"
    bits: int = 3
    rank: int = 0
    group: int = 64
    seed: int = 0
    pre_rope: bool = False
    pack_path: str = ""
    budget: float = 0.0
    dec_quant: str = "fp32"
    payload_quant: str = "rtn"


# arm pairs (K arm, V arm) that have a fused CUDA decode path in this library
FUSED_PAIRS = {
    ("lowrank_rtn_channel", "turboquant_mse_perhead"): "k2b",
    ("rtn_token", "rtn_token"): "rtn",
    ("rtn_channel", "rtn_token"): "rtn",
    ("spectral", "turboquant_mse_perhead"): "spectral",
}
