"""Pins the numpy oracle against vectors the bmx reference produced (tests/golden).

Integer and elementwise stages must be identical; stages that contain a reduction the
reference leaves to BLAS (projection, K = rank sum, row norms, attention) are held to a
tolerance that is written next to each check.
"""

import math

import numpy as np
import pytest

from oracle import bmx_oracle as O
from tests.helpers import full_rope, golden


def test_codebooks_and_flush_schedule():
    c = golden("consts")
    assert np.array_equal(c["cb2"], O.GAUSSIAN_CODEBOOK[2])
    assert np.array_equal(c["cb3"], O.GAUSSIAN_CODEBOOK[3])
    for S, W, g, want in c["flush_kat"]:
        assert O.compute_flush_schedule(int(S), int(W), int(g)) == int(want)
    # bmx tests/test_chunked_attention.py:72-77
    assert O.compute_flush_schedule(100, 32, 16) == 64
    assert O.compute_flush_schedule(40, 32, 16) == 0
    assert O.compute_flush_schedule(20, 32, 16) == 0
    assert O.compute_flush_schedule(160, 32, 1) == 128


@pytest.mark.parametrize("arm,bits,g", [("rtn_token", 2, 32), ("rtn_token", 4, 32), ("rtn_channel", 4, 32),
                                        ("rtn_channel", 2, 64), ("rtn_token", 4, 64)])
def test_rtn_arms_bit_exact(arm, bits, g):
    c = golden("codec")
    tag = f"{arm}_b{bits}_g{g}"
    p, bpe = O.quantize_packed(arm, c["M"], bits=bits, group=g)
    assert np.array_equal(p["Q_int"], c[tag + "_Q"])
    assert np.array_equal(p["scale"], c[tag + "_scale"])
    assert np.array_equal(O.dequant_packed(arm, p, group=g), c[tag + "_deq"])
    assert bpe == float(c[tag + "_bpe"]) == bits + 16.0 / g
    qmax = 2 ** (bits - 1) - 1
    assert p["Q_int"].dtype == np.int8 and p["Q_int"].min() >= -qmax - 1 and p["Q_int"].max() <= qmax


def test_fwht_bit_exact_and_involution():
    c = golden("codec")
    assert np.array_equal(O.fwht(c["fwht_in"]), c["fwht_out"])
    np.testing.assert_allclose(O.fwht(O.fwht(c["fwht_in"])), c["fwht_in"], atol=2e-6)
    # bmx tests/test_quant.py:9-14: rows of the identity give the Sylvester matrix / sqrt(d)
    H = O.fwht(np.eye(16, dtype=np.float32))
    S = np.array([[1.0]])
    while S.shape[0] < 16:
        S = np.block([[S, S], [S, -S]])
    np.testing.assert_allclose(H, S / 4.0, atol=1e-7)


@pytest.mark.parametrize("bits", [2, 3])
def test_turboquant_perhead(bits):
    c, k = golden("codec"), golden("consts")
    signs = k["signs_d128_s0"]
    p, bpe = O.quantize_packed("turboquant_mse_perhead", c["M"], bits=bits, h_heads=2, signs=signs)
    # the row norm is a reduction: fp16-rounded norms may differ in a few rows, and an index
    # can move only where the rotated value sits on a decision boundary
    assert (p["norms"] != c[f"tq_b{bits}_norms"]).mean() < 0.01
    assert (p["indices"] != c[f"tq_b{bits}_idx"]).mean() < 1e-3
    assert bpe == float(c[f"tq_b{bits}_bpe"]) == bits + 16.0 * 2 / 256
    # dequant from the REFERENCE's stored fields is elementwise: bit-exact
    ref = {"indices": c[f"tq_b{bits}_idx"], "norms": c[f"tq_b{bits}_norms"], "bits": bits, "h": 2}
    assert np.array_equal(O.dequant_packed("turboquant_mse_perhead", ref, signs=signs), c[f"tq_b{bits}_deq"])


@pytest.mark.parametrize("rank", [16, 32])
def test_lowrank_rtn_channel(rank):
    c = golden("codec")
    t = f"lr{rank}"
    p, bpe = O.quantize_packed("lowrank_rtn_channel", c[t + "_M"], bits=3, group=64, rank=rank,
                               svd_factors=(c[t + "_Us_in"], c[t + "_Vb"]))
    assert np.array_equal(p["Us"], c[t + "_Us"]) and np.array_equal(p["V"], c[t + "_V"])
    # L = Us V^T is a BLAS sum over `rank` terms: codes may move at rounding ties only
    assert (p["res_Q_int"] != c[t + "_res_Q_int"]).mean() < 1e-3
    np.testing.assert_allclose(p["res_scale"], c[t + "_res_scale"], rtol=1e-5)
    assert p["res_Q_int"].min() >= -3 and p["res_Q_int"].max() <= 3
    assert math.isclose(bpe, float(c[t + "_bpe"]), rel_tol=1e-12)
    ref = {k: c[f"{t}_{k}"] for k in ("Us", "V", "res_Q_int", "res_scale")}
    np.testing.assert_allclose(O.dequant_packed("lowrank_rtn_channel", ref, group=64), c[t + "_deq"], atol=2e-6)


def test_bit_packing_exact_inverse():
    c = golden("codec")
    assert np.array_equal(O.pack_codes(c["u2"], 2), c["u2_packed"])
    assert np.array_equal(O.pack_codes(c["u4"], 4), c["u4_packed"])
    assert np.array_equal(O.pack_signed_codes(c["s3"], 3), c["s3_packed"])
    assert np.array_equal(O.pack_signed_codes(c["s4"], 4), c["s4_packed"])
    assert np.array_equal(O.unpack_codes(c["u2_packed"], 2, 64), c["u2"])
    assert np.array_equal(O.unpack_codes(c["u4_packed"], 4, 64), c["u4"])
    assert np.array_equal(O.unpack_signed_codes(c["s3_packed"], 3, 64), c["s3"])
    assert np.array_equal(O.unpack_signed_codes(c["s4_packed"], 4, 64), c["s4"])
    with pytest.raises(AssertionError):
        O.pack_codes(c["u2"], 3)
    with pytest.raises(AssertionError):
        O.pack_signed_codes(c["s4"], 3)  # out of the signed 3-bit range


def _k2b_blocks(c, signs):
    """Rebuild block dicts from the reference's own stacked bytes (3 pages, h_kv = 2)."""
    P, C, blk = c["k2b_stack_us"].shape[0], 256, 128
    kb, vb = [], []
    for i in range(P):
        kp = {"Us": c["k2b_stack_us"][i].astype(np.float32), "V": c["k2b_stack_vfac"][i].astype(np.float32),
              "res_Q_int": O.unpack_signed_codes(c["k2b_stack_res_int_packed"][i], 3, blk),
              "res_scale": c["k2b_stack_res_scale"][i].astype(np.float32)[..., None]}
        vp = {"indices": O.unpack_codes(c["k2b_stack_v_idx_packed"][i], 2, C),
              "norms": c["k2b_stack_v_norm"][i].astype(np.float32), "bits": 2, "h": 2}
        kb.append((kp, i * blk, (i + 1) * blk))
        vb.append((vp, i * blk, (i + 1) * blk))
    return kb, vb


def test_k2b_stack_builder_and_decode():
    c, k = golden("decode"), golden("consts")
    signs = k["signs_d128_s0"]
    kb, vb = _k2b_blocks(c, signs)
    st = O.build_kv_stacked_k2b([b[0] for b in kb], [b[0] for b in vb], h_kv=2, blk=128, d=128)
    for name in ("us", "vfac", "res_scale", "v_norm", "res_int_packed", "v_idx_packed"):
        assert np.array_equal(st[name], c["k2b_stack_" + name]), name
    cos = full_rope(c["rope_cos_f32"]).astype(np.float16).astype(np.float32)
    sin = full_rope(c["rope_sin_f32"]).astype(np.float16).astype(np.float32)
    kw = dict(k_arm="lowrank_rtn_channel", v_arm="turboquant_mse_perhead", group=64, k_pre_rope=True,
              rope_cos=cos, rope_sin=sin, n_q_groups=4, scale=1.0 / math.sqrt(128), v_signs=signs)
    # the stacks hold fp16 res_scale; the reference's block dicts hold fp32 ones, so allow the
    # difference that rounding makes: 1e-3 of the largest output
    out = O.chunked_dequant_attention(c["q"], kb, vb, k_tail=c["k_tail"], v_tail=c["v_tail"], **kw)
    ref = c["k2b_out_chunked"]
    assert np.abs(out - ref).max() <= 1e-3 * np.abs(ref).max()
    naive = O.naive_dense_attention(c["q"], kb, vb, k_tail=c["k_tail"], v_tail=c["v_tail"], **kw)
    assert np.abs(naive - c["k2b_out_naive"]).max() <= 1e-3 * np.abs(ref).max()
    out_nt = O.chunked_dequant_attention(c["q"], kb, vb, k_tail=None, v_tail=None, **kw)
    assert np.abs(out_nt - c["k2b_out_chunked_notail"]).max() <= 1e-3 * np.abs(ref).max()


def test_rtn_decode_and_stacks():
    c = golden("decode")
    T, blk = c["rtn_k"].shape[0], 128
    kb_c, kb_t, vb = [], [], []
    for p0 in range(0, T, blk):
        kb_c.append((O.quantize_packed("rtn_channel", c["rtn_k"][p0:p0 + blk], bits=4, group=32)[0], p0, p0 + blk))
        kb_t.append((O.quantize_packed("rtn_token", c["rtn_k"][p0:p0 + blk], bits=4, group=32)[0], p0, p0 + blk))
        vb.append((O.quantize_packed("rtn_token", c["k2b_v"][p0:p0 + blk], bits=2, group=32)[0], p0, p0 + blk))
    kc, vc, ks, vs = O.build_kv_stacked_packed([b[0] for b in kb_t], [b[0] for b in vb], h_kv=2, blk=blk, d=128, group=32)
    for a, name in ((kc, "kc"), (vc, "vc"), (ks, "ks"), (vs, "vs")):
        assert np.array_equal(a, c["rtn_stack_" + name]), name
    kw = dict(v_arm="rtn_token", group=32, k_pre_rope=False, rope_cos=None, rope_sin=None,
              k_tail=c["k_tail"], v_tail=c["v_tail"], n_q_groups=4, scale=1.0 / math.sqrt(128))
    # same stored values on both sides; only the float32 summation order differs: 2e-5 relative
    o1 = O.chunked_dequant_attention(c["q"], kb_c, vb, k_arm="rtn_channel", **kw)
    assert np.abs(o1 - c["rtn_ct_out_chunked"]).max() <= 2e-5 * np.abs(o1).max()
    o2 = O.chunked_dequant_attention(c["q"], kb_t, vb, k_arm="rtn_token", **kw)
    assert np.abs(o2 - c["rtn_tt_out_chunked"]).max() <= 2e-5 * np.abs(o2).max()


def test_tail_partial_and_merge():
    c = golden("decode")
    q_kv = c["q"][:, 0, :].reshape(2, 4, 128)
    acc, m, l = O.tail_partial(q_kv, c["k_tail"], c["v_tail"], 1.0 / math.sqrt(128))
    np.testing.assert_allclose(acc, c["tail_acc"], rtol=2e-5, atol=2e-6)
    np.testing.assert_allclose(m, c["tail_m"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(l, c["tail_l"], rtol=2e-6)
    # bmx tests/test_decode_finalize.py: one split reduces to acc / lse; two halves merge to the whole
    np.testing.assert_allclose(O.merge_partials(acc[None], m[None], l[None]), acc / l[..., None], rtol=1e-6)
    a1, m1, l1 = O.tail_partial(q_kv, c["k_tail"][:, :20], c["v_tail"][:, :20], 1.0 / math.sqrt(128))
    a2, m2, l2 = O.tail_partial(q_kv, c["k_tail"][:, 20:], c["v_tail"][:, 20:], 1.0 / math.sqrt(128))
    merged = O.merge_partials(np.stack([a1, a2]), np.stack([m1, m2]), np.stack([l1, l2]))
    np.testing.assert_allclose(merged, acc / l[..., None], rtol=2e-5, atol=2e-6)


def test_spectral_codec():
    c = golden("spectral")
    bits = c["bits"]
    assert set(int(b) for b in bits) <= set(O.SPECTRAL_TIERS)
    np.testing.assert_array_equal(O.int8_decoder_roundtrip(c["E"], bits), c["dec8"])
    p = O.spectral_quantize_packed(c["M"], c["E"], bits, 64)
    for key in p:
        ref = c["p_" + key]
        if key.endswith("_codes"):
            # Y = M @ enc is a BLAS product: codes move only at rounding ties
            assert p[key].shape == ref.shape and (p[key] != ref).mean() < 5e-3, key
        else:
            np.testing.assert_allclose(p[key], ref, rtol=1e-4)
    refp = {k[2:]: c[k] for k in c.files if k.startswith("p_")}
    deq = O.spectral_dequant_packed(refp, c["dec8"], bits, 64)
    assert np.abs(deq - c["deq"]).max() <= 1e-5 * np.abs(c["deq"]).max()
