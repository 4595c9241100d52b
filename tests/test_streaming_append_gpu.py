"""Quantize-on-append through the layer state: token-by-token appends onto a prefix flush whole pages on
the reference's schedule, each token is quantized once from its pristine source, and the committed
prefix never changes afterwards (bmx: tests/test_streaming_cache.py:255-366 are the properties)."""

import math

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O

pytestmark = pytest.mark.gpu
D = 128


@pytest.mark.parametrize("page,dtype", [(128, torch.bfloat16), (64, torch.float16)])
def test_token_by_token_equals_bulk_and_prefix_is_frozen(page, dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables
    from bmx_b200.schedule import compute_flush_schedule

    dev = torch.device("cuda:0")
    B, h_kv, G, rank, group, W = 3, 2, 4, 32, 64, 128
    prefix, steps = 3 * page + 17, 2 * page + 5
    T = prefix + steps
    gen = torch.Generator().manual_seed(31)
    basis = torch.zeros(h_kv * D, rank)
    for h in range(h_kv):
        Q, _ = torch.linalg.qr(torch.randn(D, rank, generator=gen))
        basis[h * D:(h + 1) * D] = Q
    coef = torch.randn(B, h_kv, T, rank, generator=gen) * torch.arange(1, rank + 1).float() ** -1.5
    k_pre = (torch.einsum("bhtr,hcr->bhtc", coef, basis.view(h_kv, D, rank)) + 0.1 * torch.randn(B, h_kv, T, D, generator=gen))
    k_pre, v = k_pre.to(dtype).to(dev), torch.randn(B, h_kv, T, D, generator=gen).to(dtype).to(dev)
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)
    k_post = apply_rope(k_pre.float(), cos[:T], sin[:T]).to(dtype)
    geom = K.k2b_geom(h_kv, G, page, rank, group, h_kv)

    def fresh():
        st = K2bLayerState(geom, B, 2 * page, W, dev, cos.half(), sin.half())  # small pool: must grow
        st.set_basis(basis.to(dev))
        return st

    # streaming: prefix in one call, then one token per step
    st = fresh()
    st.append(k_pre[:, :, :prefix], k_post[:, :, :prefix], v[:, :, :prefix])
    assert st.committed == compute_flush_schedule(prefix, W, page)
    snap = None
    for t in range(prefix, T):
        st.append(k_pre[:, :, t:t + 1], k_post[:, :, t:t + 1], v[:, :, t:t + 1])
        assert st.committed == compute_flush_schedule(t + 1, W, page) and st.seq_len() == t + 1
        assert W <= st.tail_len < W + page
        if snap is None and st.committed > compute_flush_schedule(prefix, W, page):
            n0 = compute_flush_schedule(prefix, W, page) // page  # pages that existed before the first new flush
            snap = (n0, {a: x.clone() for a, x in K.k2b_export_stacks(st.pool, st.page_table[:, :n0].contiguous().view(-1)).items()})
    # bulk: everything in one call
    bulk = fresh()
    bulk.append(k_pre, k_post, v)
    assert bulk.committed == st.committed == compute_flush_schedule(T, W, page) and bulk.tail_len == st.tail_len
    n_pg = st.committed // page
    a = K.k2b_export_stacks(st.pool, st.page_table[:, :n_pg].contiguous().view(-1))
    b = K.k2b_export_stacks(bulk.pool, bulk.page_table[:, :n_pg].contiguous().view(-1))
    for name in a:
        assert torch.equal(a[name], b[name]), f"{name}: token-by-token and bulk appends wrote different bytes"
    # the committed prefix is bitwise frozen
    n0, before = snap
    after = K.k2b_export_stacks(st.pool, st.page_table[:, :n0].contiguous().view(-1))
    for name in before:
        assert torch.equal(before[name], after[name]), f"{name}: committed pages changed after later appends"
    assert torch.equal(st.k_win[:, :, : st.tail_len], bulk.k_win[:, :, : st.tail_len])
    # the window holds the last tokens, fp16-exact, and a decode over the state matches the oracle
    assert torch.equal(st.v_win[:, :, : st.tail_len], v[:, :, T - st.tail_len:].half())
    q = (torch.randn(B, h_kv * G, D, generator=gen) / math.sqrt(D)).half().to(dev)
    out = st.decode(q).float().cpu().numpy()
    ex = {n: x.cpu().numpy() for n, x in a.items()}
    basis16 = basis.half().float().numpy()
    Vb = np.zeros((h_kv * D, h_kv * rank), np.float32)
    for h in range(h_kv):
        Vb[h * D:(h + 1) * D, h * rank:(h + 1) * rank] = basis16[h * D:(h + 1) * D]
    signs = K.hadamard_signs(D, 0).numpy()
    c16, s16 = cos.half().float().cpu().numpy(), sin.half().float().cpu().numpy()
    for s in range(B):
        kb, vb = [], []
        for p in range(n_pg):
            i = s * n_pg + p
            kp = {"Us": np.concatenate([ex["us"][i, h].astype(np.float32) for h in range(h_kv)], 1), "V": Vb,
                  "res_Q_int": O.unpack_signed_codes(ex["res_int_packed"][i], 3, page),
                  "res_scale": ex["res_scale"][i].astype(np.float32)[..., None]}
            vp = {"indices": O.unpack_codes(ex["v_idx_packed"][i], 2, h_kv * D), "norms": ex["v_norm"][i].astype(np.float32),
                  "bits": 2, "h": h_kv}
            kb.append((kp, p * page, (p + 1) * page))
            vb.append((vp, p * page, (p + 1) * page))
        ref = O.chunked_dequant_attention(
            q[s].float().cpu().numpy()[:, None, :], kb, vb, k_arm="lowrank_rtn_channel", v_arm="turboquant_mse_perhead",
            group=group, k_pre_rope=True, rope_cos=c16, rope_sin=s16,
            k_tail=st.k_win[s, :, : st.tail_len].float().cpu().numpy(), v_tail=st.v_win[s, :, : st.tail_len].float().cpu().numpy(),
            n_q_groups=G, scale=1.0 / math.sqrt(D), v_signs=signs)[:, 0, :]
        err = np.abs(out[s] - ref).max(-1) / np.abs(ref).max(-1)
        assert np.all(err <= 2e-3), float(err.max())


@pytest.mark.parametrize("zero_copy,room", [(True, 3), (False, 3), (True, 8)])
def test_decode_step_graph_equals_eager_steps(zero_copy, room):
    """The captured step replayed token after token gives the outputs and the state of append() + decode() called per
    token, across flushes and a pool that grows.  zero_copy: the ingest kernel reads the pinned staging buffer itself and
    the merge kernel stores into the pinned output; otherwise copy nodes move both."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import DecodeStepGraph, K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables

    dev = torch.device("cuda:0")
    B, h_kv, G, rank, group, W, page = 2, 2, 4, 16, 64, 32, 128
    prefix, steps = 2 * page + 40, 2 * page + 9
    T = prefix + steps
    gen = torch.Generator().manual_seed(41)
    basis = torch.zeros(h_kv * D, rank)
    for h in range(h_kv):
        Q, _ = torch.linalg.qr(torch.randn(D, rank, generator=gen))
        basis[h * D:(h + 1) * D] = Q
    coef = torch.randn(B, h_kv, T, rank, generator=gen) * torch.arange(1, rank + 1).float() ** -1.5
    k_pre = (torch.einsum("bhtr,hcr->bhtc", coef, basis.view(h_kv, D, rank)) + 0.1 * torch.randn(B, h_kv, T, D, generator=gen))
    k_pre, v = k_pre.half().to(dev), torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)
    k_post = apply_rope(k_pre.float(), cos[:T], sin[:T]).half()
    qs = (torch.randn(steps, B, h_kv * G, D, generator=gen) / math.sqrt(D)).half()
    geom = K.k2b_geom(h_kv, G, page, rank, group, h_kv)

    def fresh():
        st = K2bLayerState(geom, B, room * page, W, dev, cos.half(), sin.half())  # room for 3 pages: the fourth makes it grow
        st.set_basis(basis.to(dev))
        st.append(k_pre[:, :, :prefix], k_post[:, :, :prefix], v[:, :, :prefix])
        return st

    eager, graphed = fresh(), fresh()
    nq, nk = B * h_kv * G * D, B * h_kv * D
    hin = torch.empty(nq + 3 * nk, dtype=torch.float16).pin_memory()
    hout = torch.empty(B, h_kv * G, D, dtype=torch.float16).pin_memory()
    stepper = DecodeStepGraph(graphed, hin, hout, zero_copy=zero_copy)
    assert stepper.zero_copy == zero_copy
    replays = 0
    for i in range(steps):
        t = prefix + i
        eager.append(k_pre[:, :, t:t + 1], k_post[:, :, t:t + 1], v[:, :, t:t + 1])
        ref = eager.decode(qs[i].to(dev))
        hin[:nq] = qs[i].reshape(-1)
        hin[nq:nq + nk] = k_post[:, :, t].reshape(-1).cpu()
        hin[nq + nk:nq + 2 * nk] = v[:, :, t].reshape(-1).cpu()
        hin[nq + 2 * nk:] = k_pre[:, :, t].reshape(-1).cpu()
        had_graph = stepper.graph is not None and stepper._captured_for == stepper._key()
        stepper.step()
        torch.cuda.current_stream().synchronize()
        replays += int(had_graph and stepper._captured_for == stepper._key())
        assert graphed.committed == eager.committed and graphed.tail_len == eager.tail_len
        assert int(graphed.tail_len_dev[0]) == graphed.tail_len
        assert torch.equal(hout, ref.cpu()), f"step {i}"
    K.check_status(graphed.workspace)
    assert replays > steps // 2, "most steps must have gone through the captured graph"
    assert graphed.committed // page >= 4, "two pages were committed during the run (with room for 3, the pool had to grow)"
    assert torch.equal(graphed.n_pages_dev.cpu(), eager.n_pages_dev.cpu())
    if zero_copy:  # flush steps are graphs too: the first one that fits the pool runs for real and is captured, later ones replay
        assert stepper.flush_graph is not None
        assert stepper.flush_replays == (1 if room == 8 else 0)


@pytest.mark.parametrize("kind", ["k2b", "spectral"])
def test_state_dict_round_trip_continues_bit_equal(kind):
    """A layer state saved with state_dict(), serialized, and loaded into a fresh state decodes and keeps appending
    exactly like the original (pools are compacted to the used slots on the way)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import io

    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState, SpectralLayerState
    from bmx_b200.rope import default_rope_tables

    dev = torch.device("cuda:0")
    B, h_kv, G, W, page = 2, 2, 4, 32, 128
    T = 3 * page + 50 + 140
    gen = torch.Generator().manual_seed(51)
    k_pre = torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    k_post = torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    v = torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)
    if kind == "k2b":
        geom = K.k2b_geom(h_kv, G, page, 16, 64, h_kv)
        basis = torch.cat([torch.linalg.qr(torch.randn(D, 16, generator=gen))[0] for _ in range(h_kv)], 0)

        def fresh(max_tokens):
            return K2bLayerState(geom, B, max_tokens, W, dev, cos.half(), sin.half())
    else:
        enc = torch.stack([torch.linalg.qr(torch.randn(D, D, generator=gen))[0] for _ in range(h_kv)])
        bits = torch.tensor([8] * 8 + [4] * 40 + [2] * 48 + [0] * 32, dtype=torch.int32).repeat(h_kv, 1)
        pack = K.SpectralPackDev(enc, enc.clone(), bits, page=128, group=64, device=dev)

        def fresh(max_tokens):
            return SpectralLayerState(pack, G, B, max_tokens, W, dev, cos.half(), sin.half())

    a = fresh(8 * page)
    if kind == "k2b":
        a.set_basis(basis)
    n0 = 3 * page + 50
    a.append(k_pre[:, :, :n0], k_post[:, :, :n0], v[:, :, :n0])
    buf = io.BytesIO()
    torch.save(a.state_dict(), buf)
    buf.seek(0)
    b = fresh(page)  # a smaller pool: loading must grow it
    b.load_state_dict(torch.load(buf))
    assert (b.committed, b.tail_len) == (a.committed, a.tail_len)
    q = (torch.randn(B, h_kv * G, D, generator=gen) / math.sqrt(D)).half().to(dev)
    assert torch.equal(a.decode(q), b.decode(q))
    for t in range(n0, T):  # crosses a flush
        a.append(k_pre[:, :, t:t + 1], k_post[:, :, t:t + 1], v[:, :, t:t + 1])
        b.append(k_pre[:, :, t:t + 1], k_post[:, :, t:t + 1], v[:, :, t:t + 1])
    assert a.committed == b.committed == 4 * page
    assert torch.equal(a.decode(q), b.decode(q))
    K.check_status(b.workspace)


def test_decode_step_graph_on_a_spectral_state():
    """The graph step drives the spectral layer state as well (two pools, fused spectral decode)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import DecodeStepGraph, SpectralLayerState
    from bmx_b200.rope import default_rope_tables

    dev = torch.device("cuda:0")
    B, h_kv, G, W, page = 2, 2, 4, 32, 128
    prefix, steps = page + 60, page + 20
    T = prefix + steps
    gen = torch.Generator().manual_seed(61)
    k_pre = torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    k_post = torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    v = torch.randn(B, h_kv, T, D, generator=gen).half().to(dev)
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)
    enc = torch.stack([torch.linalg.qr(torch.randn(D, D, generator=gen))[0] for _ in range(h_kv)])
    bits = torch.tensor([8] * 8 + [5] * 8 + [4] * 32 + [3] * 16 + [2] * 40 + [0] * 24, dtype=torch.int32).repeat(h_kv, 1)
    pack = K.SpectralPackDev(enc, enc.clone(), bits, page=128, group=64, device=dev)

    def fresh():
        st = SpectralLayerState(pack, G, B, 2 * page, W, dev, cos.half(), sin.half())
        st.append(k_pre[:, :, :prefix], k_post[:, :, :prefix], v[:, :, :prefix])
        return st

    eager, graphed = fresh(), fresh()
    nq, nk = B * h_kv * G * D, B * h_kv * D
    hin = torch.empty(nq + 3 * nk, dtype=torch.float16).pin_memory()
    hout = torch.empty(B, h_kv * G, D, dtype=torch.float16).pin_memory()
    stepper = DecodeStepGraph(graphed, hin, hout)
    qs = (torch.randn(steps, B, h_kv * G, D, generator=gen) / math.sqrt(D)).half()
    for i in range(steps):
        t = prefix + i
        eager.append(k_pre[:, :, t:t + 1], k_post[:, :, t:t + 1], v[:, :, t:t + 1])
        ref = eager.decode(qs[i].to(dev))
        hin[:nq] = qs[i].reshape(-1)
        hin[nq:nq + nk] = k_post[:, :, t].reshape(-1).cpu()
        hin[nq + nk:nq + 2 * nk] = v[:, :, t].reshape(-1).cpu()
        hin[nq + 2 * nk:] = k_pre[:, :, t].reshape(-1).cpu()
        stepper.step()
        torch.cuda.current_stream().synchronize()
        assert (graphed.committed, graphed.tail_len) == (eager.committed, eager.tail_len)
        assert torch.equal(hout, ref.cpu()), f"step {i}"
    K.check_status(graphed.workspace)
    assert stepper.graph is not None and graphed.committed == 2 * page
