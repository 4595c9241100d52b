"""Fused decode over a K4 spectral key cache (per-head packs) + Hadamard / 2-bit Lloyd values, through the C
ABI, against the oracle's chunked dequant-attention on the SAME stored pages: the oracle dequantizes the
exported tier containers with the float32 decoder, applies RoPE with float32 tables and attends in float32
(what bmx's chunked path does for this codec pair)."""

import math

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O

pytestmark = pytest.mark.gpu

D = 128


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def make_pack(seed, h_kv, tier_counts):
    """Per-head orthogonal encoders, a power-law spectrum and bit widths by variance rank; tier_counts maps
    bits -> number of directions (the rest get 0 bits)."""
    g = torch.Generator().manual_seed(seed)
    enc, bits = [], []
    for h in range(h_kv):
        Q, R = torch.linalg.qr(torch.randn(D, D, generator=g))
        enc.append(Q * torch.sign(torch.diagonal(R)))
        by_rank = []
        for b in sorted(tier_counts, reverse=True):
            by_rank += [b] * tier_counts[b]
        by_rank += [0] * (D - len(by_rank))
        perm = torch.randperm(D, generator=g)  # direction perm[i] has variance rank i
        bh = torch.zeros(D, dtype=torch.int32)
        bh[perm] = torch.tensor(by_rank, dtype=torch.int32)
        bits.append((bh, perm))
    return torch.stack(enc), bits


def make_keys(seed, n_seq, T, enc, bits):
    g = torch.Generator().manual_seed(seed)
    h_kv = enc.shape[0]
    k = torch.empty(n_seq, h_kv, T, D)
    for h in range(h_kv):
        perm = bits[h][1]
        lam = torch.empty(D)
        lam[perm] = torch.arange(1, D + 1).float() ** -1.2
        z = torch.randn(n_seq, T, D, generator=g) * lam.sqrt() * 4.0
        k[:, h] = z @ enc[h].T  # enc orthogonal: Y = K @ enc = z
    return k.half().contiguous()


def _case(dev, *, n_seq, h_kv, G, group, tier_counts, pages_per_seq, tail_lens, seed, tail_cap=256, dec8=False):
    from bmx_b200 import kernels as K

    max_pages = max(pages_per_seq)
    T = max(max_pages, 1) * 128
    enc, bits_perm = make_pack(seed, h_kv, tier_counts)
    bits = torch.stack([b for b, _ in bits_perm])
    dec = enc.clone()
    if dec8:
        dec = torch.stack([torch.from_numpy(O.int8_decoder_roundtrip(enc[h].numpy(), bits[h].numpy())) for h in range(h_kv)])
    pack = K.SpectralPackDev(enc, dec, bits, page=128, group=group, device=dev)
    gen = torch.Generator().manual_seed(seed + 1)
    k = make_keys(seed + 2, n_seq, T, enc, bits_perm)
    v = torch.randn(n_seq, h_kv, T, D, generator=gen).half()
    n_slots = n_seq * max(max_pages, 1) + 3
    kpool, vpool = pack.new_pool(n_slots), K.vblock_pool(h_kv, n_slots, dev)
    perm = torch.randperm(n_slots, generator=gen)
    table = perm[: n_seq * max(max_pages, 1)].view(n_seq, max(max_pages, 1)).to(torch.int32)
    signs, cb = K.hadamard_signs(D, 0), torch.tensor(K.GAUSSIAN_CODEBOOK[2])
    slots = table.reshape(-1).contiguous().to(dev)
    if max_pages > 0:
        K.spectral_append(pack, kpool, k.to(dev), slots, max_pages)
        K.vblock_append(vpool, v.to(dev), signs.to(dev), cb.to(dev), slots, max_pages)
    cos, sin = O.default_rope_tables(500000.0, D, T + tail_cap + 128)
    q = (torch.randn(n_seq, h_kv * G, D, generator=gen) / math.sqrt(D)).half()
    k_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half()
    v_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half()
    n_pages_t = torch.tensor(pages_per_seq, dtype=torch.int32)
    tail_t = torch.tensor(tail_lens, dtype=torch.int32)
    ws = K.spectral_decode_workspace(pack, G, n_seq)
    out = torch.empty(n_seq, h_kv * G, D, dtype=torch.float32, device=dev)
    scale = 1.0 / math.sqrt(D)
    K.spectral_decode(pack, G, kpool, vpool, q.to(dev), table.to(dev), n_pages_t.to(dev), max_pages,
                      torch.from_numpy(cos.astype(np.float16)).to(dev), torch.from_numpy(sin.astype(np.float16)).to(dev),
                      k_tail.to(dev), v_tail.to(dev), tail_t.to(dev), K.v_lut_tensor(K.GAUSSIAN_CODEBOOK[2], dev),
                      signs.to(dev), scale, ws, out=out)
    torch.cuda.synchronize()
    K.check_status(ws)
    # ---- oracle on the same stored pages ----
    ref = np.zeros((n_seq, h_kv * G, D), np.float32)
    cosf, sinf = cos.astype(np.float32), sin.astype(np.float32)
    for s in range(n_seq):
        npg = pages_per_seq[s]
        kb, vb = [], []
        if npg:
            sl = table[s, :npg].contiguous().to(dev)
            deq = K.spectral_dequant_pages(pack, kpool, sl, want_codes=True, want_k=False)
            vidx, vnorm = K.vblock_export(vpool, sl)
            vidx, vnorm = vidx.cpu().numpy(), vnorm.cpu().numpy()
            for p in range(npg):
                Mh = []
                for h in range(h_kv):
                    d = {a: t.cpu().numpy() for a, t in K.spectral_tier_dict(pack, deq["codes"][p, h], deq["scales"][p, h], h).items()}
                    Mh.append(O.spectral_dequant_packed(d, dec[h].numpy(), bits[h].numpy(), group))
                kb.append(({"fp16": np.concatenate(Mh, axis=1)}, p * 128, (p + 1) * 128))
                vp = {"indices": O.unpack_codes(vidx[p], 2, h_kv * D), "norms": vnorm[p].astype(np.float32), "bits": 2, "h": h_kv}
                vb.append((vp, p * 128, (p + 1) * 128))
        tl = tail_lens[s]
        ref[s] = O.chunked_dequant_attention(
            q[s].float().numpy()[:, None, :], kb, vb, k_arm="fp16", v_arm="turboquant_mse_perhead", group=group,
            k_pre_rope=True, rope_cos=cosf, rope_sin=sinf,
            k_tail=k_tail[s, :, :tl].float().numpy() if tl else None,
            v_tail=v_tail[s, :, :tl].float().numpy() if tl else None,
            n_q_groups=G, scale=scale, v_signs=signs.numpy())[:, 0, :]
    return out.cpu().numpy(), ref


def _assert_attn_close(out, ref, tol=2e-3):
    err = np.abs(out - ref).max(axis=-1)
    den = np.abs(ref).max(axis=-1)
    assert np.all(np.isfinite(out))
    assert np.all(err <= tol * den), f"worst relative error {float((err / den).max()):.3e}"


TIERS_A = {8: 5, 6: 7, 5: 13, 4: 19, 3: 22, 2: 33}        # ragged tier sizes: octets that mix widths
TIERS_B = {8: 8, 4: 40, 2: 48}                             # whole octets per tier
TIERS_C = {3: 128}                                         # one tier only, every direction carries bits


def test_value_blocks_match_oracle_containers():
    dev = _dev()
    from bmx_b200 import kernels as K

    g = torch.Generator().manual_seed(5)
    h_kv = 3
    v = torch.randn(2, h_kv, 256, D, generator=g).half()
    signs, cb = K.hadamard_signs(D, 0), torch.tensor(K.GAUSSIAN_CODEBOOK[2])
    vpool = K.vblock_pool(h_kv, 6, dev)
    slots = torch.tensor([4, 1, 0, 5], dtype=torch.int32, device=dev)
    K.vblock_append(vpool, v.to(dev), signs.to(dev), cb.to(dev), slots, 2)
    idx, norm = K.vblock_export(vpool, slots)
    idx, norm = idx.cpu().numpy(), norm.cpu().numpy()
    for s in range(2):
        for pg in range(2):
            M = v[s, :, pg * 128:(pg + 1) * 128].permute(1, 0, 2).reshape(128, h_kv * D).float().numpy()
            ind, nrm = O.turboquant_perhead_pack(M, 2, signs.numpy(), h_kv)
            got = O.unpack_codes(idx[2 * s + pg], 2, h_kv * D)
            assert (got != ind).mean() < 2e-3          # float32 Hadamard sums in another order: boundary ties only
            np.testing.assert_array_equal(norm[2 * s + pg], nrm.astype(np.float16))


@pytest.mark.parametrize("tiers,group,G,dec8", [(TIERS_A, 64, 4, False), (TIERS_B, 32, 8, False), (TIERS_C, 128, 2, False),
                                                (TIERS_A, 64, 4, True)])
def test_spectral_decode_matches_oracle(tiers, group, G, dec8):
    dev = _dev()
    out, ref = _case(dev, n_seq=2, h_kv=2, G=G, group=group, tier_counts=tiers, pages_per_seq=[5, 3], tail_lens=[37, 200],
                     seed=11, dec8=dec8)
    _assert_attn_close(out, ref)


def test_spectral_decode_random_geometries():
    """Sixteen geometries with random tier tables (widths 8/6/5/4/3/2 in ragged counts, the rest 0 bits), scale groups,
    KV heads (3 included), query heads per KV head, ragged page counts and window lengths around the 64/128/256 edges."""
    import random

    rng, dev, worst = random.Random(9), _dev(), 0.0
    for c in range(16):
        left, tiers = D, {}
        for b in (8, 6, 5, 4, 3, 2):
            if left > 0 and rng.random() < 0.7:
                tiers[b] = rng.randint(1, max(1, left // 2))
                left -= tiers[b]
        tiers = tiers or {4: 32}
        n_seq = rng.randint(1, 5)
        pages = [rng.choice([0, 1, 2, 3, 5, 9, 17]) for _ in range(n_seq)]
        tails = [rng.choice([0, 1, 63, 64, 65, 127, 128, 129, 255, 256]) for _ in range(n_seq)]
        tails = [max(t, 1) if p == 0 else t for p, t in zip(pages, tails)]  # a sequence holds at least one token
        cfg = dict(n_seq=n_seq, h_kv=rng.choice([1, 2, 3, 4, 8]), G=rng.choice([1, 2, 4, 8]), group=rng.choice([32, 64, 128]),
                   tier_counts=tiers, pages_per_seq=pages, tail_lens=tails, seed=3000 + c, dec8=rng.random() < 0.3)
        out, ref = _case(dev, **cfg)
        try:
            _assert_attn_close(out, ref)
        except AssertionError as e:
            raise AssertionError(f"{cfg}: {e}") from None
        worst = max(worst, float((np.abs(out - ref).max(-1) / np.abs(ref).max(-1)).max()))
    print(f"worst relative error over 16 geometries {worst:.2e}")


def test_spectral_decode_ragged_and_many_ranges():
    dev = _dev()
    # empty sequences, no window, more (sequence, head) ranges than CTAs can take one each
    out, ref = _case(dev, n_seq=5, h_kv=2, G=4, group=64, tier_counts=TIERS_A, pages_per_seq=[0, 7, 1, 0, 2],
                     tail_lens=[5, 0, 256, 1, 3], seed=23)
    _assert_attn_close(out, ref)
    out, ref = _case(dev, n_seq=48, h_kv=4, G=4, group=64, tier_counts=TIERS_B, pages_per_seq=[1] * 48, tail_lens=[0] * 48, seed=29)
    _assert_attn_close(out, ref)


def test_spectral_decode_many_tiles_per_cta():
    dev = _dev()
    # ~7.5 tiles per CTA on 148 SMs: the stage ring wraps and ranges span CTAs
    out, ref = _case(dev, n_seq=2, h_kv=1, G=4, group=64, tier_counts=TIERS_B, pages_per_seq=[600, 520], tail_lens=[11, 0], seed=31)
    _assert_attn_close(out, ref)


def test_spectral_sequence_split_partials_merge_to_the_whole():
    """One sequence cut into two states (the second starts at a later rotary position and owns the window): their
    partial states merged by bmxk_merge_partials equal the whole sequence decoded at once (the multi-GPU sequence
    split, both parts on one GPU here)."""
    dev = _dev()
    from bmx_b200 import kernels as K
    from bmx_b200.engine import SpectralLayerState
    from bmx_b200.rope import default_rope_tables

    h_kv, G, W, n_pg = 2, 4, 64, 12
    enc, bits_perm = make_pack(71, h_kv, TIERS_A)
    bits = torch.stack([b for b, _ in bits_perm])
    pack = K.SpectralPackDev(enc, enc.clone(), bits, page=128, group=64, device=dev)
    T = n_pg * 128 + W
    gen = torch.Generator().manual_seed(72)
    k_pre = make_keys(73, 1, T, enc, bits_perm).to(dev)
    k_post = torch.randn(1, h_kv, T, D, generator=gen).half().to(dev)
    v = torch.randn(1, h_kv, T, D, generator=gen).half().to(dev)
    q = (torch.randn(1, h_kv * G, D, generator=gen) / math.sqrt(D)).half().to(dev)
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)

    def state(first, count, window):
        st = SpectralLayerState(pack, G, 1, max(count, 1) * 128, W, dev, cos.half(), sin.half())
        sl = slice(first * 128, (first + count) * 128)
        slots = st.page_table[0, :count].contiguous()
        K.spectral_append(pack, st.kpool, k_pre[:, :, sl].contiguous(), slots, count)
        K.vblock_append(st.vpool, v[:, :, sl].contiguous(), st.signs, st.codebook, slots, count)
        st.committed = count * 128
        st.n_pages_dev.fill_(count)
        if window:
            st.k_win[:, :, :W] = k_post[:, :, n_pg * 128:]
            st.v_win[:, :, :W] = v[:, :, n_pg * 128:]
            st.tail_len = W
            st.tail_len_dev.fill_(W)
        return st

    whole = state(0, n_pg, True).decode(q, out=torch.empty(1, h_kv * G, D, dtype=torch.float32, device=dev))
    parts = []
    for first, count, window in ((0, 5, False), (5, 7, True)):
        part = torch.empty(h_kv * G, 130, dtype=torch.float32, device=dev)
        state(first, count, window).decode(q, partial_out=part, pos_offset=first * 128)
        parts.append(part)
    merged = K.merge_partials(torch.stack(parts), out=torch.empty(h_kv * G, D, dtype=torch.float32, device=dev))
    torch.cuda.synchronize()
    err = (merged - whole[0]).abs().max(dim=-1).values / whole[0].abs().max(dim=-1).values
    assert float(err.max()) < 1e-5, float(err.max())


def test_spectral_decode_parity_at_benchmark_context():
    """One sequence of 16384 committed tokens (the context of the spectral workload), two KV heads: the bar stays 2e-3
    against the oracle on the same stored pages although the accumulators of the decoder product are fp16."""
    dev = _dev()
    out, ref = _case(dev, n_seq=1, h_kv=2, G=4, group=64, tier_counts=TIERS_A, pages_per_seq=[128], tail_lens=[128], seed=43)
    err = np.abs(out - ref).max(axis=-1) / np.abs(ref).max(axis=-1)
    print(f"spectral T=16384: worst relative error {float(err.max()):.3e}")
    _assert_attn_close(out, ref)
