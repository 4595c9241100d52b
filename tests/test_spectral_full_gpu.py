"""K4 spectral keys with ONE encoder over all KV heads (the pack shape bmx fits): the chunked route of
engine.FullSpectralLayerState against the oracle's full-width codec (bmx: src/bmx/cache/spectral.py:765-839) and against
a one-shot dense attention over the same stored pages."""

import math

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O

pytestmark = pytest.mark.gpu
D = 128


def _state(dev, *, h_kv=2, G=4, n_seq=2, n_pages=3, tail=41, seed=5, chunk_pages=2):
    from bmx_b200.engine import FullSpectralLayerState
    from bmx_b200.rope import apply_rope

    g = torch.Generator().manual_seed(seed)
    C, W = h_kv * D, 64
    enc, _ = torch.linalg.qr(torch.randn(C, C, generator=g))
    tiers = [8] * 10 + [6] * 20 + [5] * 20 + [4] * 40 + [3] * 50 + [2] * 70 + [0] * (C - 210)
    bits = torch.tensor(tiers, dtype=torch.int32)[torch.randperm(C, generator=g)]
    T = n_pages * 128 + tail
    cos, sin = (torch.from_numpy(t.astype(np.float16)).to(dev) for t in O.default_rope_tables(500000.0, D, T + 256))
    st = FullSpectralLayerState(enc, enc.clone(), bits, 64, G, n_seq, T + 256, W, dev, cos, sin, chunk_pages=chunk_pages)
    k_pre = (torch.randn(n_seq, h_kv, T, D, generator=g) * torch.linspace(0.3, 2.0, D)).half()
    v = torch.randn(n_seq, h_kv, T, D, generator=g).half()
    k_post = apply_rope(k_pre.to(dev).float(), cos[:T].float(), sin[:T].float()).half()
    # filled by hand, so that the number of committed pages and the window length are what the case asks for
    st._commit_pages(k_pre.to(dev), v.to(dev), n_pages)
    st.k_win[:, :, :tail], st.v_win[:, :, :tail] = k_post[:, :, n_pages * 128:], v[:, :, n_pages * 128:].to(dev)
    st.tail_len = tail
    st.tail_len_dev.fill_(tail)
    return st, enc, bits, k_pre, v, (cos, sin)


def test_full_width_codec_matches_the_oracle():
    """Codes and scales of every direction against the oracle's spectral_quantize_packed on the full (S, C) matrix: the
    encoder product is a float32 GEMM in another summation order, so codes may differ at rounding ties only; the
    dequantized keys of the stored fields equal the oracle's decode of the same fields."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K

    dev = torch.device("cuda:0")
    st, enc, bits, k_pre, _, _ = _state(dev)
    h_kv, C = 2, 256
    for seq in range(2):
        for pg in range(3):
            M = k_pre[seq, :, pg * 128:(pg + 1) * 128].permute(1, 0, 2).reshape(128, C).float().numpy()
            want = O.spectral_quantize_packed(M, enc.numpy(), bits.numpy(), 64)
            slot = st.page_table[seq, pg:pg + 1].contiguous()
            ex = K.spectral_dequant_pages(st.pack, st.kpool, slot)
            codes = ex["codes"][0].reshape(C, 128).cpu().numpy()    # direction d = 128 g + j is row j of pseudo-head g
            scales = ex["scales"][0].reshape(C, 2).cpu().numpy()
            n_diff = n_all = 0
            for b, cols in O.tier_columns(bits.numpy()).items():
                ref_codes = O.unpack_tier_codes(want[f"t{b}_codes"], b, 128)
                n_diff += int((codes[cols] != ref_codes).sum())
                n_all += ref_codes.size
                assert np.abs(codes[cols].astype(np.int32) - ref_codes.astype(np.int32)).max() <= 1, "a differing code is the neighbouring level"
                # the step is refined from the codes (ten rounds): a group in which a code moved at a tie ends at a slightly
                # different step, every other group at the same one
                rel = np.abs(scales[cols] - want[f"t{b}_scale"][..., 0]) / want[f"t{b}_scale"][..., 0]
                assert rel.max() <= 1e-2 and (rel > 2e-4).mean() <= 0.02, (b, float(rel.max()), float((rel > 2e-4).mean()))
            assert n_diff <= 5e-3 * n_all, (n_diff, n_all)
            # stored fields -> keys: Y_hat @ dec^T, against the oracle's decode of OUR fields
            mine = {}
            for b, cols in O.tier_columns(bits.numpy()).items():
                mine[f"t{b}_codes"] = O.pack_tier_codes(codes[cols].astype(np.int8), b)
                mine[f"t{b}_scale"] = scales[cols][..., None].astype(np.float32)
            ref_k = O.spectral_dequant_packed(mine, enc.numpy(), bits.numpy(), 64)           # (128, C)
            kd, _ = st._dense_chunk(pg, pg + 1)
            got = kd[seq].permute(1, 0, 2).reshape(128, C).cpu().numpy()
            assert np.abs(got - ref_k).max() <= 2e-5 * np.abs(ref_k).max()


@pytest.mark.parametrize("chunk_pages", [1, 2, 64])
def test_chunked_decode_equals_one_shot_attention(chunk_pages):
    """The running softmax over page chunks + window equals a single softmax over all dequantized keys and values."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.rope import apply_rope

    dev = torch.device("cuda:0")
    st, _, _, _, _, (cos, sin) = _state(dev, chunk_pages=chunk_pages)
    g = torch.Generator().manual_seed(77)
    q = (torch.randn(2, 8, D, generator=g) / math.sqrt(D)).half().to(dev)
    out = st.decode(q).float()
    kd, vd = st.dense_pages()
    Tc = st.committed
    k_all = torch.cat([apply_rope(kd, cos[:Tc].float(), sin[:Tc].float()), st.k_win[:, :, : st.tail_len].float()], 2)
    v_all = torch.cat([vd, st.v_win[:, :, : st.tail_len].float()], 2)
    s = torch.einsum("bhgd,bhtd->bhgt", q.float().view(2, 2, 4, D), k_all) * st.sm_scale
    ref = torch.einsum("bhgt,bhtd->bhgd", torch.softmax(s, -1), v_all).reshape(2, 8, D)
    err = float(((out - ref).abs().amax(-1) / ref.abs().amax(-1)).max())
    print(f"chunk_pages={chunk_pages}: worst relative error {err:.3e}")
    assert err <= 2e-3  # the result is rounded to fp16
    with pytest.raises(NotImplementedError):
        st.decode(q, partial_out=torch.empty(1, device=dev))
