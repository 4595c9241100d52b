"""Spectral pack files for per-head packs, in bmx's container: one safetensors file with `layer{i}.enc`,
`layer{i}.dec`, `layer{i}.lam`, `layer{i}.bits_b{budget:g}` and a JSON sidecar `<path>.json` carrying tiers, group
and budgets (bmx: save_pack_file / load_packs, src/bmx/cache/spectral.py:1081-1164).

bmx fits one encoder over all heads, (C, C) with C = h_kv * 128; the fused kernels here take one 128 x 128
encoder per head.  Both shapes load: a per-head file stores (h_kv, 128, 128) tensors; a bmx file whose encoder and
decoder are block diagonal over heads gives per-head packs (the blocks are taken out, SpectralHeadPacks: fused
decode kernel); one that mixes heads is returned whole (SpectralFullPack: chunked route).
The decoder's int8 storage option is the same per-column round trip as bmx's (src/bmx/cache/spectral.py:913-943).
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from .packed_streaming import SpectralFullPack, SpectralHeadPacks

HEAD_DIM = 128
TIERS = (0, 2, 3, 4, 5, 6, 8)


def int8_decoder_roundtrip(dec: torch.Tensor, bits: torch.Tensor, tier_threshold: int | None = None) -> torch.Tensor:
    """Per-column symmetric int8 with an fp16 scale, applied to the decoder columns (directions) that carry bits,
    optionally only those at or below a tier; float32 in, float32 out.  dec: (..., 128 channels, 128 directions),
    bits: (..., 128)."""
    dec = dec.float()
    gate = bits != 0
    if tier_threshold is not None:
        gate = gate & (bits <= tier_threshold)
    scale = (dec.abs().amax(dim=-2) / 127.0).clamp_min(1e-12).half().float()  # per direction
    rt = (dec / scale.unsqueeze(-2)).round().clamp(-127, 127) * scale.unsqueeze(-2)
    return torch.where(gate.unsqueeze(-2), rt, dec)


def save_head_packs(path: str | Path, packs: dict[int, SpectralHeadPacks], budget: float, lam: dict[int, torch.Tensor] | None = None,
                    meta: dict | None = None) -> None:
    """Writes per-head packs of every layer under one budget label.  All layers must share the scale group."""
    from safetensors.torch import save_file

    groups = {p.group for p in packs.values()}
    assert len(groups) == 1, "all layers of a pack file share one scale group"
    tensors = {}
    for i, p in packs.items():
        tensors[f"layer{i}.enc"] = p.enc.contiguous()
        tensors[f"layer{i}.dec"] = p.dec.contiguous()
        tensors[f"layer{i}.lam"] = (lam[i] if lam is not None else torch.zeros(p.bits.shape)).float().contiguous()
        tensors[f"layer{i}.bits_b{budget:g}"] = p.bits.to(torch.int32).contiguous()
    save_file(tensors, str(path))
    sidecar = {"tiers": list(TIERS), "group": groups.pop(), "budgets": [budget], "per_head": True}
    if meta:
        assert not (set(meta) & set(sidecar)), "meta keys collide with sidecar keys"
        sidecar.update(meta)
    Path(str(path) + ".json").write_text(json.dumps(sidecar))


def _blocks(M: torch.Tensor, h_kv: int, name: str) -> torch.Tensor | None:
    """(h_kv*128, h_kv*128) block-diagonal matrix -> (h_kv, 128, 128); None when the matrix mixes heads."""
    C = h_kv * HEAD_DIM
    if M.shape != (C, C):
        raise ValueError(f"{name}: shape {tuple(M.shape)} is neither (h_kv, 128, 128) nor ({C}, {C})")
    blocks = torch.stack([M[h * HEAD_DIM:(h + 1) * HEAD_DIM, h * HEAD_DIM:(h + 1) * HEAD_DIM] for h in range(h_kv)])
    off = M.clone()
    for h in range(h_kv):
        off[h * HEAD_DIM:(h + 1) * HEAD_DIM, h * HEAD_DIM:(h + 1) * HEAD_DIM] = 0
    return blocks if float(off.abs().max()) == 0.0 else None


def load_head_packs(path: str | Path, budget: float, h_kv: int, dec_quant: str = "fp32") -> dict:
    """Per-layer per-head packs for one budget.  dec_quant: "fp32", "int8" (every direction with bits) or "int8_t{T}"
    (directions with at most T bits), as in bmx's CacheCodecSpec.dec_quant (src/bmx/cache/specs.py:12-91).
    Raises KeyError with the available budgets if `budget` is not in the file."""
    from safetensors.torch import load_file

    sidecar = json.loads(Path(str(path) + ".json").read_text())
    if budget not in sidecar["budgets"]:
        raise KeyError(f"budget {budget} not in pack file; available: {sidecar['budgets']}")
    assert set(sidecar["tiers"]) <= set(TIERS), f"tiers {sidecar['tiers']} outside {TIERS}"
    if dec_quant == "fp32":
        quant, thr = False, None
    elif dec_quant == "int8":
        quant, thr = True, 8  # every direction with bits is at most 8: the blanket round trip (bmx: spectral.py:1234-1235)
    elif dec_quant.startswith("int8_t") and dec_quant[6:].isdigit():
        quant, thr = True, int(dec_quant[6:])
    else:
        raise NotImplementedError(f"dec_quant={dec_quant!r}: supported are fp32, int8, int8_t<T>")
    tensors = load_file(str(path))
    layers = sorted({int(k.split(".")[0].removeprefix("layer")) for k in tensors if "." in k})
    out = {}
    for i in layers:
        enc, dec, bits = tensors[f"layer{i}.enc"], tensors[f"layer{i}.dec"], tensors[f"layer{i}.bits_b{budget:g}"]
        if enc.dim() == 2:
            eb, db = _blocks(enc.float(), h_kv, f"layer{i}.enc"), _blocks(dec.float(), h_kv, f"layer{i}.dec")
            if eb is None or db is None:  # one encoder over all heads, as bmx fits them: kept whole
                dec = dec.float()
                if quant:
                    dec = int8_decoder_roundtrip(dec, bits.reshape(-1), thr)
                out[i] = SpectralFullPack(enc.float(), dec, bits.reshape(-1), group=int(sidecar["group"]), tiers=tuple(sidecar["tiers"]),
                                          dec_tier=thr if quant else None)
                continue
            enc, dec, bits = eb, db, bits.reshape(h_kv, HEAD_DIM)
        if enc.shape != (h_kv, HEAD_DIM, HEAD_DIM) or bits.shape != (h_kv, HEAD_DIM):
            raise ValueError(f"layer{i}: pack shapes {tuple(enc.shape)} / {tuple(bits.shape)} do not fit h_kv={h_kv}")
        if quant:
            dec = int8_decoder_roundtrip(dec, bits, thr)
        out[i] = SpectralHeadPacks(enc, dec, bits, group=int(sidecar["group"]), tiers=tuple(sidecar["tiers"]), dec_tier=thr if quant else None)
    return out
