"""Flush schedule and bits-per-entry accounting shared by the cache classes (host side, pure Python)."""

from __future__ import annotations


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
