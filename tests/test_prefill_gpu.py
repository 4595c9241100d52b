"""Paged dequant-prefill: causal attention of a block of query positions over committed k2b pages + the fp16 window, page
by page in shared memory, against the oracle's dequantize-everything attention with the same causal mask
(bmx: src/bmx/cache/chunked_attention.py:320-395 is the route it replaces; :254-317 the oracle)."""

import math

import numpy as np
import pytest
import torch

from oracle import bmx_oracle as O
from tests.test_k2b_gpu import blocks_from_export, make_k2b_inputs, rope_tables, to_np

pytestmark = pytest.mark.gpu
D = 128


@pytest.fixture(params=["tcgen05", "mma.sync"])
def prefill_kernel(request):
    """Both kernels behind bmxk_k2b_prefill, chosen process-wide for the test and put back afterwards."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K

    K.k2b_prefill_select(0 if request.param == "tcgen05" else 1)
    yield request.param
    K.k2b_prefill_select(0)


def _case(*, n_seq, h_kv, G, rank, per_head, group, n_pages, tail, n_q, seed):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope

    dev = torch.device("cuda:0")
    page, W = 128, 64
    T = n_pages * page + tail
    k_pre, v, basis = make_k2b_inputs(seed, n_seq, h_kv, T, rank, per_head)
    cos16, sin16 = rope_tables(T + 256)
    cos, sin = torch.from_numpy(cos16).to(dev), torch.from_numpy(sin16).to(dev)
    geom = K.k2b_geom(h_kv, G, page, rank, group, h_kv if per_head else 1)
    st = K2bLayerState(geom, n_seq, T + 256, W, dev, cos, sin)
    st.set_basis(basis.to(dev))
    k_post = apply_rope(k_pre.to(dev).float(), cos[:T].float(), sin[:T].float()).half()
    # the state is filled by hand so that the window length is whatever the case asks for
    if n_pages:
        K.k2b_append(st.pool, k_pre.to(dev), v.to(dev), st.basis_f32, st.signs, st.codebook, st.page_table[:, :n_pages].contiguous().view(-1), n_pages)
    st.committed = n_pages * page
    st.n_pages_dev.fill_(n_pages)
    if tail:
        st.k_win[:, :, :tail], st.v_win[:, :, :tail] = k_post[:, :, n_pages * page:], v[:, :, n_pages * page:].to(dev)
    st.tail_len = tail
    st.tail_len_dev.fill_(tail)
    gen = torch.Generator().manual_seed(seed + 7)
    q = (torch.randn(n_seq, h_kv * G, n_q, D, generator=gen) / math.sqrt(D)).half()
    q_pos0 = T - n_q
    st.sm_scale = 1.0 / math.sqrt(D)
    out = st.prefill_attend(q.to(dev), q_pos0)
    assert out is not None
    torch.cuda.synchronize()
    K.check_status(st.workspace)
    out = out.float().cpu().numpy()
    # ---- oracle: dense K / V from the pages as stored, one masked softmax ----
    visible = np.arange(T)[None, :] <= (q_pos0 + np.arange(n_q))[:, None]
    basis16 = basis.half().float().numpy()
    cosf, sinf = cos16.astype(np.float32), sin16.astype(np.float32)
    ref = np.zeros_like(out)
    for s in range(n_seq):
        kb, vb = [], []
        if n_pages:
            ex = to_np(K.k2b_export_stacks(st.pool, st.page_table[s, :n_pages].contiguous()))
            for p in range(n_pages):
                kp, vp = blocks_from_export(ex, p, geom, basis16)
                kb.append((kp, p * page, (p + 1) * page))
                vb.append((vp, p * page, (p + 1) * page))
        ref[s] = O.naive_dense_attention(
            q[s].float().numpy(), kb, vb, k_arm="lowrank_rtn_channel", v_arm="turboquant_mse_perhead", group=group, k_pre_rope=True,
            rope_cos=cosf, rope_sin=sinf, k_tail=st.k_win[s, :, :tail].float().cpu().numpy() if tail else None,
            v_tail=st.v_win[s, :, :tail].float().cpu().numpy() if tail else None, n_q_groups=G, scale=1.0 / math.sqrt(D),
            v_signs=st.signs.cpu().numpy(), visible=visible)
    err = np.abs(out - ref).max(axis=-1) / np.abs(ref).max(axis=-1)
    return float(err.max()), out, ref


@pytest.mark.parametrize("h_kv,G,rank,per_head,group,n_pages,tail,n_q", [
    (2, 4, 32, True, 64, 5, 70, 710),      # whole prompt: every row, pages and window under the causal mask
    (2, 4, 16, False, 64, 3, 33, 100),     # the last 100 positions of a longer context, cross-head basis
    (1, 8, 32, True, 128, 2, 0, 256),      # no window; eight query heads per KV head
    (2, 2, 16, True, 32, 4, 128, 37),      # a ragged block of rows
    (2, 1, 32, True, 64, 1, 5, 133),       # one query head per KV head: 128 positions per CTA
    (1, 4, 32, True, 64, 0, 150, 150),     # no committed page: two window tiles only
    (1, 4, 16, True, 64, 9, 192, 500),     # the window's second tile partly filled, rows that start inside the pages
    (3, 2, 32, False, 128, 6, 1, 1),       # a single query row
])
def test_paged_prefill_matches_dense_oracle(prefill_kernel, h_kv, G, rank, per_head, group, n_pages, tail, n_q):
    err, _, _ = _case(n_seq=2, h_kv=h_kv, G=G, rank=rank, per_head=per_head, group=group, n_pages=n_pages, tail=tail, n_q=n_q, seed=51)
    print(f"paged prefill ({prefill_kernel}): worst relative error {err:.3e}")
    assert err <= 1e-3


def test_paged_prefill_random_geometries(prefill_kernel):
    """Ten geometries drawn over KV heads, query heads per KV head, rank, shared or per-head basis, residual group, page
    count (none included), window length (none, partial second tile) and the number of trailing query rows."""
    import random

    rng, worst = random.Random(17), 0.0
    for c in range(10):
        n_pages, tail = rng.choice([0, 1, 2, 3, 5, 9]), rng.choice([0, 1, 63, 64, 65, 127, 128, 129, 191, 192])
        if n_pages == 0 and tail == 0:
            tail = 40
        T = n_pages * 128 + tail
        cfg = dict(n_seq=rng.randint(1, 2), h_kv=rng.choice([1, 2, 4]), G=rng.choice([1, 2, 4, 8]), rank=rng.choice([16, 32]),
                   per_head=rng.choice([True, False]), group=rng.choice([32, 64, 128]), n_pages=n_pages, tail=tail,
                   n_q=rng.randint(1, min(T, 300)), seed=400 + c)
        shares = rng.choice([1, 2, 3, 5])  # the tcgen05 kernel also with its page walk shared out (ignored by the mma.sync kernel)
        from bmx_b200.engine import K2bLayerState

        orig = K2bLayerState.prefill_split
        K2bLayerState.prefill_split = lambda self, n_q, shares=shares: shares
        try:
            err, _, _ = _case(**cfg)
        finally:
            K2bLayerState.prefill_split = orig
        assert err <= 1e-3, (cfg, shares, err)
        worst = max(worst, err)
    print(f"paged prefill ({prefill_kernel}): worst relative error over 10 geometries {worst:.3e}")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("page,rank,per_head,group", [(128, 32, True, 64), (64, 16, False, 32), (128, 16, True, 128)])
def test_dense_route_dequantizer_equals_dequantize_rotate_cast(dtype, page, rank, per_head, group):
    """The dense prefill route's one-kernel dequantizer (keys rotated in float32, one rounding to the model's type, written
    in (batch, heads, rows, 128) with the window behind the pages) against the float32 page dequantizer + float32 rotation
    + cast.  Values: the same arithmetic in the same order, EQUAL.  Keys: the low-rank product is summed by mma.sync in
    another order (float32, ~1e-7), so a result may land on the other side of a 16-bit rounding boundary: at most one
    unit in the last place, in well under 1 % of the entries."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope

    dev = torch.device("cuda:0")
    n_seq, h_kv, n_pages, tail, W = 2, 2, 3, 37, 64
    T = n_pages * page + tail
    k_pre, v, basis = make_k2b_inputs(61, n_seq, h_kv, T, rank, per_head)
    cos16, sin16 = rope_tables(T + 256)
    cos, sin = torch.from_numpy(cos16).to(dev), torch.from_numpy(sin16).to(dev)
    st = K2bLayerState(K.k2b_geom(h_kv, 4, page, rank, group, h_kv if per_head else 1), n_seq, T + 256, W, dev, cos, sin)
    st.set_basis(basis.to(dev))
    st.append(k_pre.to(dev), apply_rope(k_pre.to(dev).float(), cos[:T].float(), sin[:T].float()).half(), v.to(dev))
    n_pg = st.committed // page
    assert n_pg >= 1 and st.tail_len > 0
    kd, vd = st.dense_kv(dtype)
    assert kd.shape == vd.shape == (n_seq, h_kv, st.seq_len(), D) and kd.dtype == dtype
    slots = st.page_table[:, :n_pg].contiguous().view(-1)
    k32, v32 = K.k2b_dequant_pages(st.pool, slots, st.basis_f16, st.signs, st.codebook)
    shp = (n_seq, n_pg * page, h_kv, D)
    k32 = apply_rope(k32.view(*shp).permute(0, 2, 1, 3), cos[: st.committed].float(), sin[: st.committed].float())
    got, want = kd[:, :, : st.committed].float(), k32.to(dtype).float()
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert bool(((got - want).abs() <= ulp * want.abs().clamp_min(2.0 ** -14)).all())
    assert float((got != want).float().mean()) < 0.01
    assert torch.equal(vd[:, :, : st.committed], v32.view(*shp).permute(0, 2, 1, 3).to(dtype))
    assert torch.equal(kd[:, :, st.committed:], st.k_win[:, :, : st.tail_len].to(dtype))
    assert torch.equal(vd[:, :, st.committed:], st.v_win[:, :, : st.tail_len].to(dtype))


@pytest.mark.parametrize("n_split", [2, 3, 7, 16])
def test_paged_prefill_split_pages_matches_oracle(n_split):
    """Few query rows against many pages, the page walk of every block shared out over n_split CTAs + the merge kernel:
    shares of unequal size, shares without any page (more shares than pages a block sees), the window in the last one."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.engine import K2bLayerState

    orig = K2bLayerState.prefill_split
    K2bLayerState.prefill_split = lambda self, n_q: n_split
    try:
        for kw in (dict(n_seq=2, h_kv=2, G=4, rank=32, per_head=True, group=64, n_pages=11, tail=70, n_q=40, seed=71),
                   dict(n_seq=1, h_kv=1, G=8, rank=16, per_head=False, group=32, n_pages=5, tail=0, n_q=300, seed=72),
                   dict(n_seq=1, h_kv=2, G=2, rank=32, per_head=True, group=128, n_pages=2, tail=150, n_q=1, seed=73)):
            err, _, _ = _case(**kw)
            assert err <= 1e-3, (n_split, kw, err)
    finally:
        K2bLayerState.prefill_split = orig


def test_prefill_split_heuristic():
    """One CTA per (block, head, sequence) unless that leaves SMs idle; then the number of shares that minimises
    (waves of CTAs) x (pages per share + set-up), at least four pages per share."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState

    dev = torch.device("cuda:0")
    cos16, sin16 = rope_tables(512)
    st = K2bLayerState(K.k2b_geom(8, 4, 128, 32, 64, 8), 1, 256, 64, dev, torch.from_numpy(cos16).to(dev), torch.from_numpy(sin16).to(dev))
    n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
    st.committed = 128 * 128
    assert st.prefill_split(8192) == 1 and st.prefill_split(32 * (n_sm // 8 + 1)) == 1      # a wave or more of whole walks
    s32 = st.prefill_split(32)                                                              # 8 CTAs: as many shares as one wave takes
    assert 8 * s32 <= n_sm and s32 == 16
    s256 = st.prefill_split(256)                                                            # 64 CTAs
    assert s256 > 1 and 64 * s256 <= n_sm or n_sm < 128
    st.committed = 128 * 9
    assert st.prefill_split(32) == 2            # 9 pages: shares of at least four
    st.committed = 128 * 5
    assert st.prefill_split(32) == 1


def test_paged_prefill_long_context_rows_near_the_end(prefill_kernel):
    """A 16384-token context and 64 query rows at its end: every page is fully visible, the window partly."""
    err, _, _ = _case(n_seq=1, h_kv=2, G=4, rank=32, per_head=True, group=64, n_pages=128, tail=90, n_q=64, seed=53)
    print(f"paged prefill ({prefill_kernel}), 16384-token context: worst relative error {err:.3e}")
    assert err <= 1e-3


def test_cache_prefill_takes_the_paged_route_and_agrees_with_the_dense_one():
    """Under a Hugging Face model the prompt's attention goes through the paged kernel when the mask is the plain causal
    one and the cache's prefill_route asks for it ("auto" asks for blocks below the measured row crossover, and for longer
    ones once the dense transient would pass its budget); the dense route (dequantize every page, SDPA) gives the same
    logits to fp16 accuracy."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.packed_streaming import PackedStreamingCache
    from bmx_b200.recipes import spec_pair
    from tests.test_hf_cache_gpu import _reference_model

    dev = torch.device("cuda:0")
    model = _reference_model(dev)
    ids = torch.randint(0, 256, (2, 700), generator=torch.Generator().manual_seed(9)).to(dev)
    k_spec, v_spec = spec_pair("k2b_ph", rank=16, group=64)
    calls = []
    orig = K2bLayerState.prefill_attend

    def run(paged):
        def spy(self, q, q_pos0, out=None):
            if not paged:
                return None
            calls.append((q.shape[2], q_pos0))
            return orig(self, q, q_pos0, out)

        K2bLayerState.prefill_attend = spy
        try:
            cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32, prefill_route="paged" if paged else "dense")
            with cache.attach(model), torch.no_grad():
                a = model(ids[:, :450], past_key_values=cache, use_cache=True).logits      # pages are committed before attention
                b = model(ids[:, 450:], past_key_values=cache, use_cache=True).logits      # a second block on top of a cache
            return torch.cat([a, b], 1).float()
        finally:
            K2bLayerState.prefill_attend = orig

    lp, ld = run(True), run(False)
    assert calls == [(450, 0), (450, 0), (250, 450), (250, 450)], calls  # two layers, two blocks; none from the dense run
    from bmx_b200.packed_streaming import PackedStreamingLayer

    # "auto": blocks of up to PAGED_MAX_ROWS rows take the paged kernel (it beats dequantize + SDPA there); longer blocks
    # take the dense route until its transient would pass DENSE_PREFILL_BUDGET
    assert PackedStreamingLayer.DENSE_PREFILL_BUDGET == 1 << 30 and PackedStreamingLayer.PAGED_MAX_ROWS == 2048
    cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32)
    n_before = len(calls)
    K2bLayerState.prefill_attend = lambda self, q, q_pos0, out=None: calls.append("auto") or orig(self, q, q_pos0, out)
    try:
        with cache.attach(model), torch.no_grad():
            la = model(ids[:, :450], past_key_values=cache, use_cache=True).logits.float()
            assert calls[n_before:] == ["auto", "auto"]                # 450 rows: paged, both layers
            PackedStreamingLayer.PAGED_MAX_ROWS = 100                  # a 250-row block now counts as long ...
            lb = model(ids[:, 450:], past_key_values=cache, use_cache=True).logits.float()
            assert calls[n_before:] == ["auto", "auto"]                # ... and is far below the budget: dense route
        cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32)
        PackedStreamingLayer.DENSE_PREFILL_BUDGET = 0                  # every committed page is over budget: paged again
        with cache.attach(model), torch.no_grad():
            model(ids[:, :450], past_key_values=cache, use_cache=True)
            assert calls[n_before:] == ["auto"] * 4
    finally:
        K2bLayerState.prefill_attend = orig
        PackedStreamingLayer.DENSE_PREFILL_BUDGET = 1 << 30
        PackedStreamingLayer.PAGED_MAX_ROWS = 2048
    assert float((torch.cat([la, lb], 1) - ld).abs().max()) < 5e-2
    diff = float((lp - ld).abs().max())
    print(f"paged vs dense prefill logits: max diff {diff:.3e}")
    # layer 2 quantizes keys and values that come out of layer 1's attention, where the two routes differ in the last fp16
    # bits, and 2-bit codes are discontinuous: a few codes move, so the bound here is looser than the kernel's own (1e-3)
    assert diff < 5e-2
