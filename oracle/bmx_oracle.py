"""CPU restatement (numpy, float32) of the bmx packed KV-cache codec and decode path.

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels: it is
imported by the tests, by the smoke check and by the CPU-baseline leg of the
benchmark, never by the product path.  Each function names the bmx source it
restates (paths relative to the bmx project root).

Parity status: PINNED.  Every function here is compared bit-for-bit (integer and
elementwise stages) or to a stated tolerance (reduction stages) against outputs of
the bmx reference itself; those outputs are the committed fixtures produced by
`tests/golden/make_golden.py`, and `tests/test_oracle_golden.py` replays them.

Conventions: matrices are (S, C) with C = h_kv * d, row = token, as in
src/bmx/cache/collect.py:42-51 (`to_matrix`).  All floating point work is float32
unless stated; `half_round` is the fp16 round trip the reference writes as
`.half().float()`.
"""

from __future__ import annotations

import math

import numpy as np

F32 = np.float32

# src/bmx/cache/codecs.py:346-380 (`gaussian_codebook`): empirical Lloyd-Max levels for
# N(0,1), 2**18 seeded samples, 40 iterations.  The reference computes them at run
# time; these are its float32 outputs (pinned by the golden fixture `codebooks`).
GAUSSIAN_CODEBOOK = {
    2: np.array(
        [-1.5194618701934814, -0.46033763885498047, 0.44421979784965515, 1.5017313957214355],
        dtype=F32,
    ),
    3: np.array(
        [
            -2.174412250518799, -1.3567343950271606, -0.7671520113945007, -0.2563295364379883,
            0.23005320131778717, 0.7372721433639526, 1.3183449506759644, 2.12149977684021,
        ],
        dtype=F32,
    ),
}


def half_round(x: np.ndarray) -> np.ndarray:
    """`x.half().float()`: round to nearest-even fp16 and widen again."""
    return np.asarray(x, dtype=F32).astype(np.float16).astype(F32)


# ---------------------------------------------------------------------------
# src/bmx/quant/rtn.py
# ---------------------------------------------------------------------------


def mse_refine_scale(G: np.ndarray, scale: np.ndarray, qmax: int, n_iter: int = 10) -> np.ndarray:
    """src/bmx/quant/rtn.py:10-20 (`_mse_refine_scale`)."""
    for _ in range(n_iter):
        Q = np.clip(np.rint(G / scale), -qmax - 1, qmax).astype(F32)
        num = (G * Q).sum(axis=-1, keepdims=True, dtype=F32)
        den = np.maximum((Q * Q).sum(axis=-1, keepdims=True, dtype=F32), F32(1e-12))
        scale = np.maximum(num / den, F32(1e-12)).astype(F32)
    return scale


def rtn_quantize_packed(W: np.ndarray, bits: int, group: int, mse_scale: bool = False):
    """src/bmx/quant/rtn.py:23-44.  (..., d) -> (int8 codes same shape, scale (..., d/g, 1)).

    Symmetric: scale = absmax.clamp_min(1e-12) / qmax, code = round_half_even(x/scale)
    clamped to [-qmax-1, qmax], qmax = 2**(bits-1) - 1.
    """
    W = np.asarray(W, dtype=F32)
    *lead, d = W.shape
    assert d % group == 0, f"dim {d} not divisible by group {group}"
    assert bits <= 8
    qmax = 2 ** (bits - 1) - 1
    G = W.reshape(*lead, d // group, group)
    scale = (np.maximum(np.abs(G).max(axis=-1, keepdims=True), F32(1e-12)) / F32(qmax)).astype(F32)
    if mse_scale:
        scale = mse_refine_scale(G, scale, qmax)
    Q = np.clip(np.rint(G / scale), -qmax - 1, qmax)
    return Q.astype(np.int8).reshape(W.shape), scale


def rtn_dequantize_packed(Q_int: np.ndarray, scale: np.ndarray, group: int) -> np.ndarray:
    """src/bmx/quant/rtn.py:47-53: code * scale, one float32 multiply."""
    *lead, d = Q_int.shape
    G = Q_int.reshape(*lead, d // group, group).astype(scale.dtype)
    return (G * scale).reshape(Q_int.shape)


# ---------------------------------------------------------------------------
# src/bmx/quant/hadamard.py
# ---------------------------------------------------------------------------


def fwht(x: np.ndarray) -> np.ndarray:
    """src/bmx/quant/hadamard.py:12-33: orthonormal FWHT over the last axis.

    Sylvester ordering, butterflies h = 1, 2, 4, ... with pos = a + b, neg = a - b, and
    one final TRUE division by float32(sqrt(d)) (not a reciprocal multiply).
    """
    x = np.asarray(x, dtype=F32)
    d = x.shape[-1]
    assert d > 0 and d & (d - 1) == 0
    y = x.reshape(-1, d).copy()
    h = 1
    while h < d:
        y = y.reshape(-1, d // (2 * h), 2, h)
        pos = y[:, :, 0, :] + y[:, :, 1, :]
        neg = y[:, :, 0, :] - y[:, :, 1, :]
        y = np.stack((pos, neg), axis=2).reshape(-1, d)
        h *= 2
    return (y / F32(d**0.5)).astype(F32).reshape(x.shape)


# ---------------------------------------------------------------------------
# src/bmx/cache/codecs.py -- packed arms on the streaming path
# ---------------------------------------------------------------------------


def scale_bits(group: int) -> float:
    """src/bmx/cache/codecs.py:79-81."""
    return 16.0 / group


def norm_bits(h: int, C: int) -> float:
    """src/bmx/cache/codecs.py:84-86."""
    return 16.0 * h / C


def factor_bits(rank: int, S: int, C: int) -> float:
    """src/bmx/cache/codecs.py:89-91."""
    return 16.0 * rank * (S + C) / (S * C)


def turboquant_perhead_pack(M: np.ndarray, bits: int, signs: np.ndarray, h: int):
    """src/bmx/cache/codecs.py:616-636 (`_turboquant_mse_perhead_packed`).

    `signs` is the +-1 vector of src/bmx/cache/codecs.py:114-124 for (d, seed); it comes
    from torch's generator, so the caller supplies it.  Returns (indices int16 (S, C),
    norms float32 (S, h), fp16-valued).
    """
    M = np.asarray(M, dtype=F32)
    S, C = M.shape
    d = C // h
    Mh = M.reshape(S, h, d)
    norms = half_round(np.maximum(np.sqrt((Mh * Mh).sum(axis=2, dtype=F32)), F32(1e-12)))
    unit = (Mh / norms[:, :, None]).astype(F32)
    rot = fwht((unit.reshape(S * h, d) * signs.astype(F32)).astype(F32)).reshape(S, h, d)
    cb = GAUSSIAN_CODEBOOK[bits]
    mid = ((cb[:-1] + cb[1:]) / F32(2)).astype(F32)
    scaled = (rot * F32(math.sqrt(d))).astype(F32)
    idx = np.searchsorted(mid, scaled.reshape(-1), side="left").astype(np.int16)
    return idx.reshape(S, C), norms


def turboquant_perhead_dequant(indices, norms, bits: int, signs: np.ndarray, h: int) -> np.ndarray:
    """src/bmx/cache/codecs.py:639-649 (`_turboquant_mse_perhead_dequant`)."""
    S, C = indices.shape
    d = C // h
    cb = GAUSSIAN_CODEBOOK[bits]
    q = (cb[indices.astype(np.int64)] / F32(math.sqrt(d))).astype(F32).reshape(S * h, d)
    rec = (fwht(q) * signs.astype(F32)).astype(F32).reshape(S, h, d)
    return (rec * np.asarray(norms, dtype=F32)[:, :, None]).astype(F32).reshape(S, C)


def lowrank_split(M: np.ndarray, Us: np.ndarray, V: np.ndarray):
    """src/bmx/cache/codecs.py:677-695 (`_lowrank_split`) with `svd_factors` given.

    Returns (Us_stored, V_stored, L, R): fp16-valued factors, L = Us V^T, R = M - L.
    The K = rank sum in L is a BLAS call in the reference; its order is not pinned.
    """
    Us_s = half_round(Us)
    V_s = half_round(V)
    L = (Us_s @ V_s.T).astype(F32)
    return Us_s, V_s, L, (np.asarray(M, dtype=F32) - L).astype(F32)


def quantize_packed(arm: str, M: np.ndarray, *, bits: int, group: int = 64, rank: int = 0,
                    svd_factors=None, h_heads: int = 0, signs: np.ndarray | None = None):
    """src/bmx/cache/codecs.py:698-796 for the arms that have a CUDA path here."""
    M = np.asarray(M, dtype=F32)
    S, C = M.shape
    if arm == "rtn_token":
        Q, sc = rtn_quantize_packed(M, bits, group)
        return {"Q_int": Q, "scale": sc}, bits + scale_bits(group)
    if arm == "rtn_channel":
        Q, sc = rtn_quantize_packed(np.ascontiguousarray(M.T), bits, group)
        return {"Q_int": Q, "scale": sc}, bits + scale_bits(group)
    if arm in ("turboquant_mse", "turboquant_mse_perhead"):
        h = h_heads if (arm == "turboquant_mse_perhead" and h_heads > 0) else 1
        idx, norms = turboquant_perhead_pack(M, bits, signs, h)
        out = {"indices": idx, "norms": norms, "bits": bits}
        if arm == "turboquant_mse_perhead":
            out["h"] = h
        return out, bits + norm_bits(h, C)
    if arm == "lowrank_rtn_channel":
        assert S % group == 0
        assert svd_factors is not None, "the oracle takes the frozen factors as input"
        Us_s, V_s, _, R = lowrank_split(M, *svd_factors)
        Q, sc = rtn_quantize_packed(np.ascontiguousarray(R.T), bits, group)
        bpe = bits + scale_bits(group) + factor_bits(rank, S, C)
        return {"Us": Us_s, "V": V_s, "res_Q_int": Q, "res_scale": sc}, bpe
    raise NotImplementedError(arm)


def dequant_packed(arm: str, packed: dict, *, group: int = 64, signs: np.ndarray | None = None):
    """src/bmx/cache/codecs.py:799-842."""
    if arm == "rtn_token":
        return rtn_dequantize_packed(packed["Q_int"], packed["scale"], group)
    if arm == "rtn_channel":
        return rtn_dequantize_packed(packed["Q_int"], packed["scale"], group).T
    if arm in ("turboquant_mse", "turboquant_mse_perhead"):
        h = packed.get("h", 1)
        return turboquant_perhead_dequant(packed["indices"], packed["norms"], packed["bits"], signs, h)
    if arm == "lowrank_rtn_channel":
        L = (packed["Us"] @ packed["V"].T).astype(F32)
        R_hat = rtn_dequantize_packed(packed["res_Q_int"], packed["res_scale"], group).T
        return (L + R_hat).astype(F32)
    raise NotImplementedError(arm)


# ---------------------------------------------------------------------------
# src/bmx/cache/triton_dequant_attention.py -- bit packing and stack builders
# ---------------------------------------------------------------------------


def pack_codes(idx: np.ndarray, bits: int) -> np.ndarray:
    """src/bmx/cache/triton_dequant_attention.py:49-83: unsigned codes, 8/bits per byte along
    the last axis, code c in byte c // per_byte at bit offset bits * (c % per_byte)."""
    assert 8 % bits == 0 and bits < 8
    per = 8 // bits
    C = idx.shape[-1]
    assert C % per == 0
    g = idx.astype(np.uint8).reshape(*idx.shape[:-1], C // per, per).astype(np.int32)
    shifts = (np.arange(per, dtype=np.int32) * bits)
    return (g << shifts).sum(axis=-1).astype(np.uint8)


def unpack_codes(packed: np.ndarray, bits: int, C: int) -> np.ndarray:
    """src/bmx/cache/triton_dequant_attention.py:86-100: exact inverse, int16 out."""
    assert 8 % bits == 0 and bits < 8
    per = 8 // bits
    assert C % per == 0 and packed.shape[-1] == C // per
    shifts = (np.arange(per, dtype=np.int32) * bits)
    codes = (packed.astype(np.int32)[..., None] >> shifts) & ((1 << bits) - 1)
    return codes.reshape(*packed.shape[:-1], C).astype(np.int16)


def pack_signed_codes(code: np.ndarray, bits: int) -> np.ndarray:
    """src/bmx/cache/triton_dequant_attention.py:103-140: two's-complement nibbles, two per
    byte along the last axis, low nibble first, whatever `bits` (<= 4) is."""
    assert 1 <= bits <= 4
    qmax = 2 ** (bits - 1) - 1
    assert int(code.min()) >= -qmax - 1 and int(code.max()) <= qmax
    N = code.shape[-1]
    assert N % 2 == 0
    nib = (code.astype(np.int32) & 0xF).reshape(*code.shape[:-1], N // 2, 2)
    return (nib[..., 0] | (nib[..., 1] << 4)).astype(np.uint8)


def unpack_signed_codes(packed: np.ndarray, bits: int, N: int) -> np.ndarray:
    """src/bmx/cache/triton_dequant_attention.py:143-165."""
    assert 1 <= bits <= 4 and N % 2 == 0 and packed.shape[-1] == N // 2
    p = packed.astype(np.int32)
    inter = np.stack([p & 0xF, (p >> 4) & 0xF], axis=-1).reshape(*packed.shape[:-1], N)
    return ((inter ^ 0x8) - 0x8).astype(np.int8)


def from_matrix(M: np.ndarray, h: int) -> np.ndarray:
    """src/bmx/cache/collect.py:48-51: (S, h*d) -> (h, S, d)."""
    S, hd = M.shape
    return M.reshape(S, h, hd // h).transpose(1, 0, 2)


def to_matrix(kv: np.ndarray) -> np.ndarray:
    """src/bmx/cache/collect.py:42-45: (h, S, d) -> (S, h*d) float32."""
    h, S, d = kv.shape
    return np.ascontiguousarray(kv.transpose(1, 0, 2)).reshape(S, h * d).astype(F32)


def build_kv_stacked_k2b(k_blocks, v_blocks, *, h_kv: int, blk: int, d: int,
                         pack_k: bool = True, pack_v: bool = True, k_bits: int = 3) -> dict:
    """src/bmx/cache/triton_dequant_attention.py:1118-1229: the byte layout the reference
    kernels read (fp16 casts of factors, scales and norms happen here)."""
    C = h_kv * d
    P = len(k_blocks)
    rank = k_blocks[0]["Us"].shape[1]
    n_kg = k_blocks[0]["res_scale"].shape[1]
    vbits = int(v_blocks[0]["bits"])
    out = {
        "us": np.zeros((P, blk, rank), np.float16),
        "vfac": np.zeros((P, C, rank), np.float16),
        "res_scale": np.zeros((P, C, n_kg), np.float16),
        "v_norm": np.zeros((P, blk, h_kv), np.float16),
        "rank": rank, "k_group": blk // n_kg,
    }
    res = np.zeros((P, C, blk // 2 if pack_k else blk), np.uint8 if pack_k else np.int8)
    vi = np.zeros((P, blk, C // (8 // vbits) if pack_v else C), np.uint8 if pack_v else np.int16)
    for i, (kp, vp) in enumerate(zip(k_blocks, v_blocks)):
        out["us"][i] = kp["Us"].astype(np.float16)
        out["vfac"][i] = kp["V"].astype(np.float16)
        out["res_scale"][i] = kp["res_scale"][..., 0].astype(np.float16)
        res[i] = pack_signed_codes(kp["res_Q_int"], k_bits) if pack_k else kp["res_Q_int"]
        out["v_norm"][i] = vp["norms"].astype(np.float16)
        vi[i] = pack_codes(vp["indices"], vbits) if pack_v else vp["indices"]
    out["res_int_packed" if pack_k else "res_int"] = res
    out["v_idx_packed" if pack_v else "v_idx"] = vi
    if pack_k:
        out["pack_k"], out["k_bits"] = True, k_bits
    if pack_v:
        out["pack_v"], out["vbits"] = True, vbits
    return out


def build_kv_stacked_packed(k_blocks, v_blocks, *, h_kv: int, blk: int, d: int, group: int,
                            v_group: int | None = None):
    """src/bmx/cache/triton_dequant_attention.py:1390-1451 (rtn_token layout on both sides):
    int8 containers (P, h_kv, blk, d) and fp16 scales (P, h_kv, blk, d // group)."""
    vg = v_group if v_group is not None else group
    P = len(k_blocks)
    kc = np.zeros((P, h_kv, blk, d), np.int8)
    vc = np.zeros((P, h_kv, blk, d), np.int8)
    ks = np.zeros((P, h_kv, blk, d // group), np.float16)
    vs = np.zeros((P, h_kv, blk, d // vg), np.float16)
    for i, (kp, vp) in enumerate(zip(k_blocks, v_blocks)):
        kc[i] = from_matrix(kp["Q_int"], h_kv)
        ks[i] = from_matrix(kp["scale"][..., 0].astype(np.float16), h_kv)
        vc[i] = from_matrix(vp["Q_int"], h_kv)
        vs[i] = from_matrix(vp["scale"][..., 0].astype(np.float16), h_kv)
    return kc, vc, ks, vs


# ---------------------------------------------------------------------------
# src/bmx/cache/rope.py
# ---------------------------------------------------------------------------


def rotate_half(x: np.ndarray) -> np.ndarray:
    """src/bmx/cache/rope.py:61-72: cat(-x[d/2:], x[:d/2])."""
    d = x.shape[-1]
    return np.concatenate((-x[..., d // 2:], x[..., : d // 2]), axis=-1)


def apply_rope(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """src/bmx/cache/rope.py:75-102: x (h, S, d), cos/sin (S, d); x*cos + rotate_half(x)*sin."""
    return x * cos[None] + rotate_half(x) * sin[None]


def default_rope_tables(theta: float, d: int, S: int, start: int = 0):
    """cos/sin (S, d) float32 for the un-scaled ("default") rotary embedding that
    src/bmx/cache/rope.py:19-58 obtains from transformers' LlamaRotaryEmbedding:
    inv_freq = theta ** -(arange(0, d, 2) / d), angle = position * inv_freq, both halves
    of the head share the angle.  Elementary functions may differ from torch's by an ulp,
    so tests that need the reference's exact table take it from the fixture instead."""
    inv = (1.0 / (F32(theta) ** (np.arange(0, d, 2, dtype=np.int64).astype(F32) / F32(d)))).astype(F32)
    pos = np.arange(start, start + S, dtype=np.int64).astype(F32)
    fr = (pos[:, None] * inv[None, :]).astype(F32)
    emb = np.concatenate((fr, fr), axis=-1)
    return np.cos(emb).astype(F32), np.sin(emb).astype(F32)


# ---------------------------------------------------------------------------
# src/bmx/cache/streaming.py and the split heuristics
# ---------------------------------------------------------------------------


def compute_flush_schedule(S: int, W: int, g: int) -> int:
    """src/bmx/cache/streaming.py:144-151."""
    return ((S - W) // g) * g if S > W else 0


def pick_num_splits(seq_len: int, blk: int, h_kv: int, n_sms: int = 132, occupancy_mult: int = 2) -> int:
    """src/bmx/cache/triton_dequant_attention.py:464-501."""
    n_blocks = max(1, (seq_len + blk - 1) // blk)
    target = max(1, occupancy_mult * n_sms // max(1, h_kv))
    target = min(target, n_blocks, 64)
    p = 1
    while p * 2 <= target:
        p *= 2
    return p


# ---------------------------------------------------------------------------
# src/bmx/cache/chunked_attention.py -- the decode oracle and its pieces
# ---------------------------------------------------------------------------


def dequant_block(packed: dict, arm: str, group: int, h_kv: int, signs=None) -> np.ndarray:
    """src/bmx/cache/chunked_attention.py:52-145 (`_dequant_block`): packed dict -> (h_kv, blk, d)."""
    M = packed["fp16"] if arm == "fp16" else dequant_packed(arm, packed, group=group, signs=signs)
    return from_matrix(np.asarray(M), h_kv)


def chunked_dequant_attention(q, k_blocks, v_blocks, *, k_arm, v_arm, group, k_pre_rope,
                              rope_cos, rope_sin, k_tail, v_tail, n_q_groups, scale,
                              v_group=None, v_signs=None, k_signs=None, dtype=F32):
    """src/bmx/cache/chunked_attention.py:478-530, decode branch (n_q == 1 or more rows, no mask).

    q (n_q_heads, n_q, d); blocks are lists of (packed, start, end).  Accumulates in
    `dtype` (the reference accumulates in q.dtype; float32 q gives the float32 oracle).
    Non-spectral order: dequantized K is cast to `dtype`, then RoPE'd with the given
    tables (fp16 tables in the packed cache, src/bmx/cache/packed_streaming.py:94-113).
    """
    q = np.asarray(q, dtype=dtype)
    n_q_heads, n_q, d = q.shape
    h_kv = n_q_heads // n_q_groups
    vg = v_group if v_group is not None else group
    acc = np.zeros((n_q_heads, n_q, d), dtype)
    m = np.full((n_q_heads, n_q, 1), -np.inf, dtype)
    lse = np.zeros((n_q_heads, n_q, 1), dtype)
    qg = q.reshape(h_kv, n_q_groups, n_q, d)

    def attend(K, V):
        nonlocal acc, m, lse
        s = (np.einsum("gpnd,gbd->gpnb", qg, K).astype(dtype) * dtype(scale)).astype(dtype)
        s = s.reshape(n_q_heads, n_q, K.shape[1])
        m_new = np.maximum(m, s.max(axis=-1, keepdims=True))
        corr = np.exp(m - m_new)
        p = np.exp(s - m_new).astype(dtype)
        lse = (lse * corr + p.sum(axis=-1, keepdims=True, dtype=dtype)).astype(dtype)
        pg = p.reshape(h_kv, n_q_groups, n_q, K.shape[1])
        av = np.einsum("gpnb,gbd->gpnd", pg, V).astype(dtype).reshape(n_q_heads, n_q, d)
        acc = (acc * corr + av).astype(dtype)
        m = m_new

    for (kp, start, end), (vp, _s, _e) in zip(k_blocks, v_blocks):
        K = dequant_block(kp, k_arm, group, h_kv, signs=k_signs).astype(dtype)
        if k_pre_rope:
            K = apply_rope(K, rope_cos[start:end], rope_sin[start:end]).astype(dtype)
        V = dequant_block(vp, v_arm, vg, h_kv, signs=v_signs).astype(dtype)
        attend(K, V)
    if k_tail is not None and k_tail.shape[1] > 0:
        attend(k_tail.astype(dtype), v_tail.astype(dtype))
    return acc / lse


def naive_dense_attention(q, k_blocks, v_blocks, *, k_arm, v_arm, group, k_pre_rope, rope_cos,
                          rope_sin, k_tail, v_tail, n_q_groups, scale, v_group=None,
                          v_signs=None, k_signs=None, dtype=F32, visible=None):
    """src/bmx/cache/chunked_attention.py:254-317: dequantize everything, one softmax.  `visible`: optional boolean
    (n_q, S) mask, True where the key may be attended (the prefill route applies the model's causal mask the same way,
    src/bmx/cache/chunked_attention.py:320-395)."""
    q = np.asarray(q, dtype=dtype)
    h_kv = q.shape[0] // n_q_groups
    vg = v_group if v_group is not None else group
    Ks, Vs = [], []
    for (kp, start, end), (vp, _s, _e) in zip(k_blocks, v_blocks):
        K = dequant_block(kp, k_arm, group, h_kv, signs=k_signs)
        if k_pre_rope:
            K = apply_rope(K, rope_cos[start:end].astype(K.dtype), rope_sin[start:end].astype(K.dtype))
        Ks.append(K.astype(dtype))
        Vs.append(dequant_block(vp, v_arm, vg, h_kv, signs=v_signs).astype(dtype))
    if k_tail is not None and k_tail.shape[1] > 0:
        Ks.append(k_tail.astype(dtype))
        Vs.append(v_tail.astype(dtype))
    K = np.repeat(np.concatenate(Ks, axis=1), n_q_groups, axis=0)
    V = np.repeat(np.concatenate(Vs, axis=1), n_q_groups, axis=0)
    s = (q @ K.transpose(0, 2, 1)) * dtype(scale)
    if visible is not None:
        s = np.where(np.asarray(visible, bool)[None], s, dtype(-np.inf))
    s = s - s.max(axis=-1, keepdims=True)
    p = np.exp(s)
    return (p / p.sum(axis=-1, keepdims=True)) @ V


def tail_partial(q_kv, k_tail, v_tail, scale: float):
    """src/bmx/cache/triton_dequant_attention.py:324-360: the fp16 window as one split.
    q_kv (h_kv, G, d); returns acc (h_kv, G, d), m (h_kv, G), lse (h_kv, G), float32."""
    qf, kf, vf = (np.asarray(a, dtype=F32) for a in (q_kv, k_tail, v_tail))
    s = np.einsum("hgd,htd->hgt", qf, kf).astype(F32) * F32(scale)
    m = s.max(axis=-1)
    p = np.exp(s - m[..., None]).astype(F32)
    return np.einsum("hgt,htd->hgd", p, vf).astype(F32), m, p.sum(axis=-1, dtype=F32)


def merge_partials(acc, m, lse):
    """src/bmx/cache/triton_dequant_attention.py:409-461 (`_fused_merge_kernel`), base e:
    m* = max_s m_s ; l = sum_s lse_s e^{m_s - m*} ; o = sum_s acc_s e^{m_s - m*} / l.
    acc (n_splits, ..., d); m, lse (n_splits, ...)."""
    acc, m, lse = (np.asarray(a, dtype=F32) for a in (acc, m, lse))
    mg = m.max(axis=0)
    w = np.exp(m - mg[None]).astype(F32)
    l = (lse * w).sum(axis=0, dtype=F32)
    o = (acc * w[..., None]).sum(axis=0, dtype=F32)
    return (o / l[..., None]).astype(F32)


# ---------------------------------------------------------------------------
# src/bmx/cache/spectral.py -- the K4 spectral key codec (packed form)
# ---------------------------------------------------------------------------

SPECTRAL_TIERS = (0, 2, 3, 4, 5, 6, 8)  # src/bmx/cache/spectral.py:423


def tier_columns(bits: np.ndarray) -> dict:
    """src/bmx/cache/spectral.py:631-645: ascending column indices per non-zero tier."""
    return {int(b): np.nonzero(bits == b)[0] for b in sorted(set(int(x) for x in bits)) if b != 0}


def pack_tier_codes(Q_int: np.ndarray, b: int) -> np.ndarray:
    """src/bmx/cache/spectral.py:703-739, quantizer "rtn": tiers 2/4 offset-binary through
    pack_codes, tier 3 signed nibbles, tiers 5/6/8 the int8 container."""
    if b in (2, 4):
        return pack_codes(Q_int.astype(np.int16) + 2 ** (b - 1), b)
    if b == 3:
        return pack_signed_codes(Q_int, b)
    return Q_int


def unpack_tier_codes(t: np.ndarray, b: int, S: int) -> np.ndarray:
    """src/bmx/cache/spectral.py:742-762."""
    if b in (2, 4):
        return (unpack_codes(t, b, S) - 2 ** (b - 1)).astype(np.int8)
    if b == 3:
        return unpack_signed_codes(t, b, S)
    return t


def spectral_quantize_packed(M, enc, bits, group: int, mse_scale: bool = True) -> dict:
    """src/bmx/cache/spectral.py:765-809: Y = M @ enc, then per tier RTN (10-step MSE scale
    refinement) along tokens on Y[:, cols].T."""
    M = np.asarray(M, dtype=F32)
    S, C = M.shape
    assert S % group == 0
    Y = (M @ np.asarray(enc, dtype=F32)).astype(F32)
    packed = {}
    for b, cols in tier_columns(bits).items():
        Q, sc = rtn_quantize_packed(np.ascontiguousarray(Y[:, cols].T), b, group, mse_scale=mse_scale)
        packed[f"t{b}_codes"] = pack_tier_codes(Q, b)
        packed[f"t{b}_scale"] = sc
    return packed


def spectral_dequant_packed(packed: dict, dec, bits, group: int) -> np.ndarray:
    """src/bmx/cache/spectral.py:812-839: scatter the tiers back, then M_hat = Y_hat @ dec^T."""
    cols_by = tier_columns(bits)
    first = next(iter(cols_by))
    S = packed[f"t{first}_scale"].shape[1] * group
    dec = np.asarray(dec, dtype=F32)
    Y = np.zeros((S, dec.shape[0]), F32)
    for b, cols in cols_by.items():
        Q = unpack_tier_codes(packed[f"t{b}_codes"], b, S)
        Y[:, cols] = rtn_dequantize_packed(Q, packed[f"t{b}_scale"], group).T
    return (Y @ dec.T).astype(F32)


def int8_decoder_roundtrip(dec: np.ndarray, bits_pc: np.ndarray, tier_threshold=None) -> np.ndarray:
    """src/bmx/cache/spectral.py:913-943: per-column symmetric int8 with an fp16 scale, applied
    to the columns that carry bits (optionally only those at or below a tier)."""
    dec = np.asarray(dec, dtype=F32)
    gate = bits_pc != 0
    if tier_threshold is not None:
        gate = gate & (bits_pc <= tier_threshold)
    out = dec.copy()
    g = dec[:, gate]
    scale = half_round(np.maximum(np.abs(g).max(axis=0) / F32(127.0), F32(1e-12)))
    out[:, gate] = (np.clip(np.rint(g / scale), -127, 127) * scale).astype(F32)
    return out
