"""Rotary-embedding tables in the form the cache keeps them: (positions, head_dim) cos/sin.

`rope_tables_from_config` goes through the model family's own rotary module, exactly as bmx does
(bmx: src/bmx/cache/rope.py:19-58), so scaled variants (llama3, yarn, ...) are inherited from the
config.  `default_rope_tables` is the un-scaled formula for callers that have no HF config.
"""

from __future__ import annotations

import torch


def default_rope_tables(theta: float, head_dim: int, n_pos: int, device="cpu", start: int = 0):
    """float32 cos/sin (n_pos, head_dim): angle = position * theta ** -(2i / head_dim), both halves alike."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.int64, device=device).float() / head_dim))
    pos = torch.arange(start, start + n_pos, dtype=torch.int64, device=device).float()
    fr = pos[:, None] * inv[None, :]
    emb = torch.cat((fr, fr), dim=-1)
    return emb.cos(), emb.sin()


def rope_tables_from_config(config, n_pos: int, start: int = 0, device=None):
    """float32 cos/sin (n_pos, head_dim) for positions [start, start + n_pos) of an HF config."""
    from transformers.models.llama.modeling_llama import LlamaRotaryEmbedding

    tc = getattr(config, "text_config", None)
    if tc is not None and hasattr(tc, "num_attention_heads"):
        config = tc
    if not hasattr(config, "rope_parameters") and not hasattr(config, "rope_theta"):
        raise ValueError(f"Config {type(config).__name__} has no rotary embedding")
    rot = LlamaRotaryEmbedding(config=config).eval()
    if device is not None:
        rot = rot.to(device)
    d = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
    x = torch.zeros(1, n_pos, d, device=device)
    pos = torch.arange(start, start + n_pos, dtype=torch.long, device=device)
    with torch.no_grad():
        cos, sin = rot(x, pos.unsqueeze(0))
    return cos.squeeze(0), sin.squeeze(0)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x (..., S, d) * cos + rotate_half(x) * sin with (S, d) tables (bmx: src/bmx/cache/rope.py:75-102)."""
    d = x.shape[-1]
    rot = torch.cat((-x[..., d // 2:], x[..., : d // 2]), dim=-1)
    return x * cos + rot * sin
