"""GPU parity of the plain-RTN path (bmx arms rtn_token / rtn_channel): every codec stage is
elementwise, so codes and fp16 scales must equal the oracle's bit for bit; attention within 2e-3."""

import math

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O
from tests.helpers import golden

pytestmark = pytest.mark.gpu
D = 128


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _inputs(seed, n_seq, h_kv, T):
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(n_seq, h_kv, T, D, generator=g)
    k[..., :4] *= 8.0  # outlier channels, as in the RTN benchmark configuration
    return k.half().contiguous(), torch.randn(n_seq, h_kv, T, D, generator=g).half().contiguous()


def _oracle_blocks(k, v, s, p, page, k_arm, kg, vg, kbits):
    Mk = O.to_matrix(k[s, :, p * page:(p + 1) * page].float().numpy())
    Mv = O.to_matrix(v[s, :, p * page:(p + 1) * page].float().numpy())
    kp, _ = O.quantize_packed(k_arm, Mk, bits=kbits, group=kg)
    vp, _ = O.quantize_packed("rtn_token", Mv, bits=2, group=vg)
    return kp, vp


@pytest.mark.parametrize("page,k_arm,kg,vg,kbits", [(128, "rtn_channel", 32, 32, 4), (128, "rtn_token", 32, 32, 4),
                                                     (64, "rtn_channel", 64, 64, 2), (64, "rtn_token", 64, 128, 3),
                                                     (128, "rtn_token", 128, 32, 4)])
def test_append_codes_and_scales_bit_exact(page, k_arm, kg, vg, kbits):
    from bmx_b200 import kernels as K
    dev = _dev()
    h_kv, n_seq, n_pg = 2, 2, 2
    k, v = _inputs(3, n_seq, h_kv, n_pg * page)
    g = K.rtn_geom(h_kv, 4, page, k_arm, kg, vg, kbits, 2)
    pool = K.RtnPool(g, 8, dev)
    slots = torch.tensor([6, 1, 3, 4], dtype=torch.int32, device=dev)
    K.rtn_append(pool, k.to(dev), v.to(dev), slots, n_pg)
    ex = {a: t.cpu().numpy() for a, t in K.rtn_export(pool, slots, dequant=True).items()}
    for s in range(n_seq):
        for p in range(n_pg):
            i = s * n_pg + p
            kp, vp = _oracle_blocks(k, v, s, p, page, k_arm, kg, vg, kbits)
            if k_arm == "rtn_token":
                assert np.array_equal(ex["k_codes"][i], O.from_matrix(kp["Q_int"], h_kv))
                assert np.array_equal(ex["k_scales"][i], O.from_matrix(kp["scale"][..., 0].astype(np.float16), h_kv))
                k16 = {"Q_int": kp["Q_int"], "scale": kp["scale"].astype(np.float16).astype(np.float32)}
            else:
                assert np.array_equal(ex["k_codes"][i], kp["Q_int"])
                assert np.array_equal(ex["k_scales"][i], kp["scale"][..., 0].astype(np.float16))
                k16 = {"Q_int": kp["Q_int"], "scale": kp["scale"].astype(np.float16).astype(np.float32)}
            assert np.array_equal(ex["v_codes"][i], O.from_matrix(vp["Q_int"], h_kv))
            assert np.array_equal(ex["v_scales"][i], O.from_matrix(vp["scale"][..., 0].astype(np.float16), h_kv))
            v16 = {"Q_int": vp["Q_int"], "scale": vp["scale"].astype(np.float16).astype(np.float32)}
            # dequant = code * (fp16-stored) scale, one float32 multiply: bit-exact
            assert np.array_equal(ex["k_deq"][i], O.dequant_packed(k_arm, k16, group=kg))
            assert np.array_equal(ex["v_deq"][i], O.dequant_packed("rtn_token", v16, group=vg))
            qmax = 2 ** (kbits - 1) - 1
            assert ex["k_codes"][i].min() >= -qmax and ex["k_codes"][i].max() <= qmax


def _decode_case(K, dev, *, page, k_arm, kg, vg, G, pages_per_seq, tail_lens, seed, h_kv=2, kbits=4):
    n_seq, max_pages, tail_cap = len(pages_per_seq), max(pages_per_seq), 256
    k, v = _inputs(seed, n_seq, h_kv, max(max_pages, 1) * page)
    g = K.rtn_geom(h_kv, G, page, k_arm, kg, vg, kbits, 2)
    n_slots = n_seq * max(max_pages, 1) + 2
    pool = K.RtnPool(g, n_slots, dev)
    gen = torch.Generator().manual_seed(seed + 1)
    table = torch.randperm(n_slots, generator=gen)[: n_seq * max(max_pages, 1)].view(n_seq, -1).to(torch.int32)
    if max_pages:
        K.rtn_append(pool, k.to(dev), v.to(dev), table.reshape(-1).contiguous().to(dev), max_pages)
    q = (torch.randn(n_seq, h_kv * G, D, generator=gen) / math.sqrt(D)).half()
    k_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half()
    v_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half()
    ws = K.rtn_workspace(g, n_seq, max_pages, dev)
    out = torch.empty(n_seq, h_kv * G, D, dtype=torch.float32, device=dev)
    scale = 1.0 / math.sqrt(D)
    K.rtn_decode(pool, q.to(dev), table.to(dev), torch.tensor(pages_per_seq, dtype=torch.int32, device=dev), max_pages,
                 k_tail.to(dev), v_tail.to(dev), torch.tensor(tail_lens, dtype=torch.int32, device=dev), scale, ws, out=out)
    torch.cuda.synchronize()
    ref = np.zeros((n_seq, h_kv * G, D), np.float32)
    for s in range(n_seq):
        kb, vb = [], []
        for p in range(pages_per_seq[s]):
            kp, vp = _oracle_blocks(k, v, s, p, page, k_arm, kg, vg, kbits)
            kp["scale"] = kp["scale"].astype(np.float16).astype(np.float32)  # the pages hold fp16 scales
            vp["scale"] = vp["scale"].astype(np.float16).astype(np.float32)
            kb.append((kp, p * page, (p + 1) * page))
            vb.append((vp, p * page, (p + 1) * page))
        tl = tail_lens[s]
        ref[s] = O.chunked_dequant_attention(
            q[s].float().numpy()[:, None, :], kb, vb, k_arm=k_arm, v_arm="rtn_token", group=kg, v_group=vg, k_pre_rope=False,
            rope_cos=None, rope_sin=None, k_tail=k_tail[s, :, :tl].float().numpy() if tl else None,
            v_tail=v_tail[s, :, :tl].float().numpy() if tl else None, n_q_groups=G, scale=scale)[:, 0, :]
    return out.cpu().numpy(), ref


def _close(out, ref, tol=2e-3):
    err, den = np.abs(out - ref).max(axis=-1), np.abs(ref).max(axis=-1)
    assert np.all(np.isfinite(out)) and np.all(err <= tol * den), f"worst relative error {float((err / den).max()):.3e}"


@pytest.mark.parametrize("page,k_arm,kg,vg,G", [(128, "rtn_channel", 32, 32, 4), (128, "rtn_token", 32, 32, 4),
                                                (64, "rtn_channel", 64, 64, 2), (64, "rtn_token", 128, 128, 8),
                                                (128, "rtn_token", 64, 32, 1)])
def test_decode_matches_oracle(page, k_arm, kg, vg, G):
    from bmx_b200 import kernels as K
    out, ref = _decode_case(K, _dev(), page=page, k_arm=k_arm, kg=kg, vg=vg, G=G, pages_per_seq=[5, 0, 3],
                            tail_lens=[37, 200, 0], seed=21)
    _close(out, ref)


def test_decode_random_geometries():
    """Sixteen geometries drawn over page, key arm, group sizes, code width, KV heads, query heads per KV head, ragged
    page counts and window lengths around the 64/128/256 edges, each against the oracle."""
    import random

    from bmx_b200 import kernels as K
    rng, dev, worst = random.Random(5), _dev(), 0.0
    for c in range(16):
        page, n_seq = rng.choice([64, 128]), rng.randint(1, 5)
        pages = [rng.choice([0, 1, 2, 3, 5, 9, 17]) for _ in range(n_seq)]
        tails = [rng.choice([0, 1, 63, 64, 65, 127, 128, 129, 255, 256]) for _ in range(n_seq)]
        tails = [max(t, 1) if p == 0 else t for p, t in zip(pages, tails)]  # a sequence holds at least one token
        cfg = dict(page=page, k_arm=rng.choice(["rtn_channel", "rtn_token"]),
                   kg=rng.choice([g for g in (32, 64, 128) if g <= page]), vg=rng.choice([32, 64, 128]),
                   G=rng.choice([1, 2, 4, 8]), pages_per_seq=pages, tail_lens=tails, seed=2000 + c,
                   h_kv=rng.choice([1, 2, 4, 8]), kbits=rng.choice([2, 3, 4]))
        out, ref = _decode_case(K, dev, **cfg)
        try:
            _close(out, ref)
        except AssertionError as e:
            raise AssertionError(f"{cfg}: {e}") from None
        worst = max(worst, float((np.abs(out - ref).max(-1) / np.abs(ref).max(-1)).max()))
    print(f"worst relative error over 16 geometries {worst:.2e}")


def test_first_baseline_config_shape():
    """Benchmark configuration 1: 8 KV heads, GQA 4, T = 4096 + 128-token window, K rtn_channel 4b, V rtn_token 2b, g = 32."""
    from bmx_b200 import kernels as K
    out, ref = _decode_case(K, _dev(), page=128, k_arm="rtn_channel", kg=32, vg=32, G=4, pages_per_seq=[32],
                            tail_lens=[128], seed=1000, h_kv=8)
    _close(out, ref)


def test_reference_golden_rtn():
    """The reference's own stacked tensors and chunked outputs (3 pages, h_kv = 2) for the same inputs."""
    from bmx_b200 import kernels as K
    dev, c = _dev(), golden("decode")
    h_kv, G, page, n_pg = 2, 4, 128, 3
    k = torch.from_numpy(O.from_matrix(c["rtn_k"], h_kv).copy())[None].half().contiguous()
    v = torch.from_numpy(O.from_matrix(c["k2b_v"], h_kv).copy())[None].half().contiguous()
    tl = c["k_tail"].shape[1]
    k_tail = torch.zeros(1, h_kv, 64, D, dtype=torch.float16)
    v_tail = torch.zeros(1, h_kv, 64, D, dtype=torch.float16)
    k_tail[0, :, :tl], v_tail[0, :, :tl] = torch.from_numpy(c["k_tail"]), torch.from_numpy(c["v_tail"])
    q = torch.from_numpy(c["q"][:, 0, :])[None].half().contiguous()
    slots = torch.arange(n_pg, dtype=torch.int32, device=dev)
    for k_arm, want in (("rtn_token", "rtn_tt_out_chunked"), ("rtn_channel", "rtn_ct_out_chunked")):
        g = K.rtn_geom(h_kv, G, page, k_arm, 32, 32, 4, 2)
        pool = K.RtnPool(g, n_pg, dev)
        K.rtn_append(pool, k.to(dev), v.to(dev), slots, n_pg)
        if k_arm == "rtn_token":
            ex = K.rtn_export(pool, slots)
            assert np.array_equal(ex["k_codes"].cpu().numpy(), c["rtn_stack_kc"])
            assert np.array_equal(ex["v_codes"].cpu().numpy(), c["rtn_stack_vc"])
            assert np.array_equal(ex["k_scales"].cpu().numpy(), c["rtn_stack_ks"])
            assert np.array_equal(ex["v_scales"].cpu().numpy(), c["rtn_stack_vs"])
        ws = K.rtn_workspace(g, 1, n_pg, dev)
        out = torch.empty(1, h_kv * G, D, dtype=torch.float32, device=dev)
        K.rtn_decode(pool, q.to(dev), slots.view(1, -1), torch.tensor([n_pg], dtype=torch.int32, device=dev), n_pg,
                     k_tail.to(dev), v_tail.to(dev), torch.tensor([tl], dtype=torch.int32, device=dev), 1.0 / math.sqrt(D), ws, out=out)
        torch.cuda.synchronize()
        _close(out.cpu().numpy(), c[want][:, 0, :][None])
