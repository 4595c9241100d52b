"""The pinned-order C restatement agrees with the numpy oracle (which follows the reference) wherever
the order of a float32 sum does not matter, and only at rounding ties where it does."""

import numpy as np

from oracle import bmx_oracle as O
from oracle import cpu_ref
from tests.helpers import golden


def test_c_restatement_vs_numpy_oracle_and_reference_vectors():
    c, k = golden("codec"), golden("consts")
    signs, cb = k["signs_d128_s0"].astype(np.float32), k["cb2"]
    M, Vb = c["lr16_M"], c["lr16_Vb"]
    out = cpu_ref.k2b_quant_page(M, c["M"], Vb, signs, cb, h_kv=2, page=128, rank=16, group=64, n_coef_heads=1)
    # coefficients: same fp16 value as the reference's stored Us except at fp16 rounding ties
    us_ref = c["lr16_Us"].astype(np.float16)
    assert (out["us"][0] != us_ref).mean() < 0.01
    ulp = np.maximum(np.abs(us_ref.astype(np.float32)), 2.0 ** -14) * 2.0 ** -10
    assert np.all(np.abs(out["us"][0].astype(np.float32) - us_ref.astype(np.float32)) <= 1.01 * ulp)
    # integer stages given the C code's own coefficients: identical to the numpy oracle up to ties in L
    p, _ = O.quantize_packed("lowrank_rtn_channel", M, bits=3, group=64, rank=16,
                             svd_factors=(out["us"][0].astype(np.float32), Vb))
    assert (p["res_Q_int"] != out["res_Q_int"]).mean() < 1e-3
    assert (p["res_scale"][..., 0].astype(np.float16) != out["res_scale"]).mean() < 1e-2
    # values against the reference's own indices and norms
    assert (out["v_idx"] != c["tq_b2_idx"]).mean() < 1e-3
    assert (out["v_norm"] != c["tq_b2_norms"].astype(np.float16)).mean() < 0.02
    assert out["res_Q_int"].min() >= -3 and out["res_Q_int"].max() <= 3 and out["v_idx"].max() <= 3
