"""The page-slot allocator (host logic, no GPU) and the multi-sequence layer state built on it (GPU)."""

import math

import pytest
import torch

from bmx_b200.paging import PageAllocator


def test_allocator_hands_out_frees_and_reuses_slots():
    a = PageAllocator(8)
    assert a.alloc("s0", 3) == [0, 1, 2] and a.alloc("s1", 2) == [3, 4] and a.in_use == 5
    assert a.alloc("s0", 1) == [5] and a.slots("s0") == [0, 1, 2, 5]
    with pytest.raises(MemoryError):
        a.alloc("s2", 3)                       # only two slots are free: nothing changes
    assert a.in_use == 6 and a.slots("s2") == []
    assert a.free("s0") == 4 and a.in_use == 2 and a.slots("s0") == []
    got = a.alloc("s2", 5)                     # the freed slots come back, lowest first
    assert sorted(got) == [0, 1, 2, 5, 6] and a.peak_in_use == 7
    a.grow(4)
    assert a.n_slots == 12 and sorted(a.alloc("s3", 5)) == [7, 8, 9, 10, 11]
    assert a.free("nobody") == 0


@pytest.mark.gpu
def test_sequences_join_leave_and_share_one_pool():
    """Three sequences of different lengths over one pool; one ends, a new one takes over its slots; every live sequence
    decodes to what a state of its own gives, and memory per sequence follows from the allocator's counts."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.paging import PagedK2bLayer
    from bmx_b200.rope import apply_rope, default_rope_tables
    from tests.test_k2b_gpu import make_k2b_inputs

    dev = torch.device("cuda:0")
    h_kv, G, D, rank, page, group, W = 2, 4, 128, 32, 128, 64, 32
    lens = {"a": 3 * page + 50, "b": 2 * page + 7, "c": 5 * page + W + 3, "d": 4 * page + 99}
    k_all, v_all, basis = make_k2b_inputs(61, len(lens), h_kv, max(lens.values()), rank, True)
    cos, sin = default_rope_tables(500000.0, D, 2048, device=dev)
    geom = K.k2b_geom(h_kv, G, page, rank, group, h_kv)
    layer = PagedK2bLayer(geom, n_slots=10, max_seqs=3, recent_window=W, device=dev, rope_cos=cos.half(), rope_sin=sin.half())
    layer.set_basis(basis)
    data = {}
    for i, (name, T) in enumerate(lens.items()):
        k_pre, v = k_all[i, :, :T].to(dev), v_all[i, :, :T].to(dev)
        data[name] = (k_pre, apply_rope(k_pre.float(), cos[:T], sin[:T]).half(), v)

    def feed(name, chunk):
        layer.add_sequence(name)
        k_pre, k_post, v = data[name]
        for t0 in range(0, k_pre.shape[1], chunk):  # in blocks, so that pages are allocated as the sequence grows
            layer.append(name, k_pre[:, t0:t0 + chunk], k_post[:, t0:t0 + chunk], v[:, t0:t0 + chunk])

    def alone(name, q):
        k_pre, k_post, v = data[name]
        st = K2bLayerState(geom, 1, 2048, W, dev, cos.half(), sin.half())
        st.set_basis(basis.to(dev))
        st.append(k_pre[None], k_post[None], v[None])
        return st.decode(q[None])[0].float()

    feed("a", 100), feed("b", 64), feed("c", 1000)
    assert layer.alloc.in_use == 3 + 1 + 5 and layer.seq_len("c") == lens["c"]
    g = torch.Generator().manual_seed(3)
    q = (torch.randn(3, h_kv * G, D, generator=g) / math.sqrt(D)).half().to(dev)
    out = layer.decode(["a", "b", "c"], q).float()
    for i, name in enumerate(("a", "b", "c")):
        ref = alone(name, q[i])
        assert float((out[i] - ref).abs().max() / ref.abs().max()) < 1e-3, name
    with pytest.raises(MemoryError):
        feed("d", 512)                          # all three rows are taken
    assert layer.drop_sequence("a") == 3 and layer.alloc.in_use == 6
    feed("d", 512)                               # takes a's row and needs 4 slots: 3 of them are a's old ones
    assert sorted(layer.alloc.slots("d"))[:3] == [0, 1, 2] and layer.alloc.in_use == 10
    out = layer.decode(["d", "c"], q[:2]).float()
    for i, name in enumerate(("d", "c")):
        ref = alone(name, q[i])
        assert float((out[i] - ref).abs().max() / ref.abs().max()) < 1e-3, name
    st = layer.memory_stats()
    assert st["slots_in_use"] == 10 and st["peak_slots_in_use"] == 10 and st["sequences"] == 3
    assert st["packed_page_bytes"] == 10 * (h_kv * 13056 + h_kv * 8192)
    assert st["bytes_per_token"] < st["dense_fp16_bytes_per_token"]
