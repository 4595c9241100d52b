"""Spectral pack files (host side, no GPU): per-head packs survive a save / load round trip in bmx's container,
a bmx-shaped file (one (C, C) encoder) gives per-head packs when it is block diagonal over heads and one whole pack
when it mixes heads, and the decoder's int8 round trip equals the oracle's."""

import json

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O


def _packs(h_kv=2, layers=2, seed=0):
    from bmx_b200.packed_streaming import SpectralHeadPacks

    g = torch.Generator().manual_seed(seed)
    tiers = [8] * 4 + [6] * 8 + [4] * 30 + [3] * 20 + [2] * 40 + [0] * 26
    out = {}
    for i in range(layers):
        enc = torch.stack([torch.linalg.qr(torch.randn(128, 128, generator=g))[0] for _ in range(h_kv)])
        bits = torch.stack([torch.tensor(tiers, dtype=torch.int32)[torch.randperm(128, generator=g)] for _ in range(h_kv)])
        out[i] = SpectralHeadPacks(enc, enc.clone(), bits, group=64)
    return out


def test_round_trip_and_budget_lookup(tmp_path):
    from bmx_b200.packs import load_head_packs, save_head_packs

    packs = _packs()
    path = tmp_path / "packs.safetensors"
    save_head_packs(path, packs, 2.5, meta={"note": "seeded"})
    side = json.loads((tmp_path / "packs.safetensors.json").read_text())
    assert side["group"] == 64 and side["budgets"] == [2.5] and side["tiers"] == [0, 2, 3, 4, 5, 6, 8] and side["note"] == "seeded"
    back = load_head_packs(path, 2.5, h_kv=2)
    assert sorted(back) == [0, 1]
    for i in packs:
        assert torch.equal(back[i].enc, packs[i].enc) and torch.equal(back[i].dec, packs[i].dec)
        assert torch.equal(back[i].bits, packs[i].bits) and back[i].group == 64
    with pytest.raises(KeyError):
        load_head_packs(path, 3.0, h_kv=2)
    with pytest.raises(ValueError):
        load_head_packs(path, 2.5, h_kv=4)


def test_bmx_shaped_file_block_diagonal_or_whole(tmp_path):
    from safetensors.torch import save_file

    from bmx_b200.packs import load_head_packs

    packs = _packs(layers=1)[0]
    C = 256
    enc = torch.zeros(C, C)
    for h in range(2):
        enc[h * 128:(h + 1) * 128, h * 128:(h + 1) * 128] = packs.enc[h]
    tensors = {"layer0.enc": enc, "layer0.dec": enc.clone(), "layer0.lam": torch.ones(C), "layer0.bits_b2.5": packs.bits.reshape(-1)}
    path = tmp_path / "fullc.safetensors"
    save_file(tensors, str(path))
    (tmp_path / "fullc.safetensors.json").write_text(json.dumps({"tiers": [0, 2, 3, 4, 5, 6, 8], "group": 64, "budgets": [2.5]}))
    back = load_head_packs(path, 2.5, h_kv=2)[0]
    assert torch.equal(back.enc, packs.enc) and torch.equal(back.bits, packs.bits)
    enc[0, 200] = 0.01  # one entry that couples two heads
    save_file(dict(tensors, **{"layer0.enc": enc}), str(path))
    from bmx_b200.packed_streaming import SpectralFullPack

    whole = load_head_packs(path, 2.5, h_kv=2)[0]
    assert isinstance(whole, SpectralFullPack) and torch.equal(whole.enc, enc) and whole.bits.shape == (C,)
    assert whole.c_used == int((packs.bits != 0).sum()) and whole.group == 64
    q8 = load_head_packs(path, 2.5, h_kv=2, dec_quant="int8")[0]
    assert q8.dec_tier == 8 and q8.dec.shape == (C, C)
    np.testing.assert_array_equal(q8.dec.numpy(), O.int8_decoder_roundtrip(tensors["layer0.dec"].numpy(), packs.bits.reshape(-1).numpy(), None))


def test_int8_decoder_round_trip_equals_oracle(tmp_path):
    from bmx_b200.packs import int8_decoder_roundtrip, load_head_packs, save_head_packs

    packs = _packs(layers=1)
    p = packs[0]
    for thr in (None, 4):
        got = int8_decoder_roundtrip(p.dec, p.bits, thr)
        for h in range(2):
            ref = O.int8_decoder_roundtrip(p.dec[h].numpy(), p.bits[h].numpy(), thr)
            np.testing.assert_array_equal(got[h].numpy(), ref)
    path = tmp_path / "p.safetensors"
    save_head_packs(path, packs, 2.5)
    assert torch.equal(load_head_packs(path, 2.5, 2, dec_quant="int8")[0].dec, int8_decoder_roundtrip(p.dec, p.bits))
    assert torch.equal(load_head_packs(path, 2.5, 2, dec_quant="int8_t4")[0].dec, int8_decoder_roundtrip(p.dec, p.bits, 4))
    with pytest.raises(NotImplementedError):
        load_head_packs(path, 2.5, 2, dec_quant="int8_tl")
