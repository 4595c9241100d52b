"""Flush schedule and bits-per-entry accounting shared by the cache classes (host side, pure Python)."""

from __future__ import annotations

import math


def compute_flush_schedule(S: int, W: int, g: int) -> int:
    """Largest multiple of g that leaves at least W recent tokens in fp16, else 0.

    Same formula and argument meaning as bmx: src/bmx/cache/streaming.py:144-151.
    """
    return ((S - W) // g) * g if S > W else 0


def scale_bits(group: int) -> float:
    """fp16 scale per `group` entries (bmx: src/bmx/cache/codecs.py:79-81)."""
    return 16.0 / group


def norm_bits(h: int, C: int) -> float:
    """fp16 norms, h per row of C channels (bmx: src/bmx/cache/codecs.py:84-86)."""
    return 16.0 * h / C


def factor_bits(rank: int, S: int, C: int) -> float:
    """fp16 low-rank factors Us (S x r) + V (C x r) per entry (bmx: src/bmx/cache/codecs.py:89-91)."""
    return 16.0 * rank * (S + C) / (S * C)


def codec_bpe(arm: str, *, bits: int, group: int, rank: int, S: int, C: int, h_heads: int = 1) -> float:
    """Bits per entry that bmx's quantize_packed reports for one page of S tokens
    (bmx: src/bmx/cache/codecs.py:720-796)."""
    if arm in ("rtn_token", "rtn_channel"):
        return bits + scale_bits(group)
    if arm == "turboquant_mse":
        return bits + norm_bits(1, C)
    if arm == "turboquant_mse_perhead":
        return bits + norm_bits(h_heads if h_heads > 0 else 1, C)
    if arm == "lowrank_rtn_channel":
        return bits + scale_bits(group) + factor_bits(rank, S, C)
    if arm == "fp16":
        return 16.0
    raise NotImplementedError(f"no packed accounting for arm {arm!r}")


def tier_bits(tiers, S: int) -> float:
    """Tier map of the spectral codec: ceil(log2(number of tiers)) bits per channel, amortized over S tokens
    (bmx: src/bmx/cache/codecs.py:94-96)."""
    return math.ceil(math.log2(len(tiers))) / S


def mixed_dec_charge(C: int, S: int, tiers, *, c_used: float, c_int8: float) -> float:
    """Per-sequence charge of a spectral pack's decoder and tier map, in bits per entry: `c_int8` of the `c_used`
    decoder columns that carry bits are held as int8 (8 bits per entry plus one fp16 scale per column), the rest as
    fp16 (bmx: src/bmx/cache/spectral.py:1036-1064)."""
    assert 0 <= c_int8 <= c_used <= C, f"need 0 <= c_int8 <= c_used <= C; got {c_int8}, {c_used}, {C}"
    int8_term = 8.0 * c_int8 / S + 16.0 * c_int8 / (S * C)
    fp16_term = 16.0 * (c_used - c_int8) / S
    return int8_term + fp16_term + tier_bits(tiers, S)


def cache_bits_per_entry(layers, k_spec) -> tuple[float, float]:
    """(bpe_k, bpe_v): blended bits per entry averaged across layers; a spectral cache that has committed pages is
    also charged its packs' decoders and tier map once per sequence (bmx: src/bmx/cache/streaming.py:154-260).
    `layers` expose bpe_k, bpe_v, _committed_S_q, get_seq_length(), _h_kv, _d_head and (spectral) _pack."""
    layers = list(layers)
    if not layers:
        return float("nan"), float("nan")
    last = layers[-1]
    bpe_k = sum(layer.bpe_k for layer in layers) / len(layers)
    bpe_v = sum(layer.bpe_v for layer in layers) / len(layers)
    if k_spec.arm == "spectral" and last._committed_S_q > 0:
        S, C = last.get_seq_length(), last._h_kv * last._d_head
        mean_c_used = sum(layer._pack.c_used for layer in layers) / len(layers)
        mean_c_int8 = sum(0 if layer._pack.dec_tier is None else layer._pack.c_int8(layer._pack.dec_tier) for layer in layers) / len(layers)
        bpe_k = bpe_k + mixed_dec_charge(C, S, last._pack.tiers, c_used=mean_c_used, c_int8=mean_c_int8)
    return bpe_k, bpe_v
