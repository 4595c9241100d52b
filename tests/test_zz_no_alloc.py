"""The decode entry point for hosts that cannot allocate device memory.

An inference server that reserved all free HBM for its page pool, or a plugin living inside another
runtime's process, has no way to hand `bmxk_k2b_decode` a freshly allocated workspace.
`bmxk_k2b_decode_static` runs the same kernels on a 2 MiB scratch array that ships inside the
library.  This test calls it through the C ABI twice in a row (the scratch keeps the first call's
contents, so the second call proves nothing stale is read) and checks both results against the
ordinary entry point, within the decode path's own 2e-3 bar; it also checks the size limit.

The file name sorts last on purpose: if this fails, every other test has already run.
"""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_decode_matches_workspace_decode_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200._lib import BmxkError
    from bmx_b200.rope import default_rope_tables

    dev = torch.device("cuda:0")
    h_kv, G, D, page, rank, group, n_seq, n_pg, tail_cap = 2, 4, 128, 128, 32, 64, 3, 4, 160
    gen = torch.Generator().manual_seed(5)
    g = K.k2b_geom(h_kv, G, page, rank, group, h_kv)
    pool = K.K2bPool(g, n_seq * n_pg, dev)
    basis = torch.zeros(h_kv * D, rank)
    for h in range(h_kv):
        Q, _ = torch.linalg.qr(torch.randn(D, rank, generator=gen))
        basis[h * D:(h + 1) * D] = Q
    k = torch.randn(n_seq, h_kv, n_pg * page, D, generator=gen).half().to(dev)
    v = torch.randn(n_seq, h_kv, n_pg * page, D, generator=gen).half().to(dev)
    signs = K.hadamard_signs(D, 0).to(dev)
    cb = torch.tensor(K.GAUSSIAN_CODEBOOK[2], device=dev)
    table = torch.arange(n_seq * n_pg, dtype=torch.int32, device=dev).view(n_seq, n_pg)
    K.k2b_append(pool, k, v, basis.to(dev), signs, cb, table.reshape(-1).contiguous(), n_pg)
    cos, sin = default_rope_tables(500000.0, D, n_pg * page + 512)
    cos, sin = cos.half().to(dev), sin.half().to(dev)
    n_pages = torch.tensor([4, 2, 3], dtype=torch.int32, device=dev)
    tail_len = torch.tensor([100, 33, 160], dtype=torch.int32, device=dev)
    k_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half().to(dev)
    v_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half().to(dev)
    lut = K.v_lut_tensor(K.GAUSSIAN_CODEBOOK[2], dev)
    b16 = basis.half().to(dev)
    scale = 1.0 / math.sqrt(D)

    def tol_check(a, b):
        a, b = a.float().cpu().numpy(), b.float().cpu().numpy()
        err = np.abs(a - b).max(axis=-1)
        assert np.all(np.isfinite(a)) and np.all(err <= 2e-3 * np.abs(b).max(axis=-1))

    for attempt in range(2):  # two calls in a row on the shared scratch, with different queries
        q = (torch.randn(n_seq, h_kv * G, D, generator=gen) / math.sqrt(D)).half().to(dev)
        ws = K.decode_workspace(g, n_seq, n_pg, dev)
        ref = torch.empty(n_seq, h_kv * G, D, dtype=torch.float32, device=dev)
        K.k2b_decode(pool, q, b16, table, n_pages, n_pg, cos, sin, k_tail, v_tail, tail_len, lut, signs, scale, ws, out=ref)
        out = torch.full((n_seq, h_kv * G, D), float("nan"), dtype=torch.float32, device=dev)
        K.k2b_decode_static(pool, q, b16, table, n_pages, n_pg, cos, sin, k_tail, v_tail, tail_len, lut, signs, scale, out)
        torch.cuda.synchronize()
        tol_check(out, ref)

    # a batch whose partial states do not fit the built-in scratch is refused, with both sizes in the message
    big_g = K.k2b_geom(64, 8, page, rank, group, 64)
    big_q = torch.zeros(64, 64 * 8, D, dtype=torch.float16, device=dev)
    with pytest.raises(BmxkError) as ei:
        K.k2b_decode_static(K.K2bPool(big_g, 1, dev), big_q, b16, table, torch.zeros(64, dtype=torch.int32, device=dev), 1,
                            cos, sin, None, None, None, lut, signs, scale,
                            torch.empty(64, 64 * 8, D, dtype=torch.float16, device=dev))
    assert "scratch" in str(ei.value) and str(K.STATIC_SCRATCH_BYTES) in str(ei.value)
