"""The decode entry point for hosts that cannot allocate device memory.

An inference server that reserved all free HBM for its page pool, or a plugin living inside another
runtime's process, has no way to hand `bmxk_k2b_decode` a freshly allocated workspace.
`bmxk_k2b_decode_static` runs the same kernels on a 2 MiB scratch array that ships inside the
library.  This test calls it through the C ABI twice in a row (the scratch keeps the first call's
contents, so the second call proves nothing stale is read) and checks both results against the
ordinary entry point and against the CPU oracle on the same stored pages, within the decode path's own
2e-3 bar; it reads the scratch's status word through `bmxk_k2b_decode_static_status` after each call,
checks that the free device memory does not move across a call, and checks the size limit.  Both page
layouts (each has its own decode kernel) and both output types are covered.

The file name sorts last on purpose: if this fails, every other test has already run.
"""

import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tol_check(a, b, what):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    err = np.abs(a - b).max(axis=-1)
    den = np.abs(b).max(axis=-1)
    assert np.all(np.isfinite(a)), what
    assert np.all(err <= 2e-3 * den), f"{what}: worst relative error {float((err / den).max()):.3e}"


@pytest.mark.parametrize("page,layout,out_dtype", [(128, 1, torch.float32), (128, 0, torch.float16), (64, 0, torch.float32)])
def test_static_scratch_decode_matches_workspace_decode_twice(page, layout, out_dtype):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200 import kernels as K
    from bmx_b200._lib import BmxkError
    from bmx_b200.rope import default_rope_tables
    from oracle import bmx_oracle as O
    from tests.test_k2b_gpu import blocks_from_export, to_np

    dev = torch.device("cuda:0")
    h_kv, G, D, rank, group, n_seq, n_pg, tail_cap = 2, 4, 128, 32, 64, 3, 4, 160
    gen = torch.Generator().manual_seed(5)
    g = K.k2b_geom(h_kv, G, page, rank, group, h_kv, layout=layout)
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
    pages_per_seq, tail_lens = [4, 2, 3], [100, 33, 160]
    n_pages = torch.tensor(pages_per_seq, dtype=torch.int32, device=dev)
    tail_len = torch.tensor(tail_lens, dtype=torch.int32, device=dev)
    k_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half().to(dev)
    v_tail = torch.randn(n_seq, h_kv, tail_cap, D, generator=gen).half().to(dev)
    lut = K.v_lut_tensor(K.GAUSSIAN_CODEBOOK[2], dev)
    b16 = basis.half().to(dev)
    scale = 1.0 / math.sqrt(D)

    def oracle(q):
        """The CPU oracle's chunked dequant-attention over the pages as stored (exported in bmx's layout)."""
        ref = np.zeros((n_seq, h_kv * G, D), np.float32)
        basis16 = basis.half().float().numpy()
        cosf, sinf = cos.float().cpu().numpy(), sin.float().cpu().numpy()
        for s in range(n_seq):
            st = to_np(K.k2b_export_stacks(pool, table[s, :pages_per_seq[s]].contiguous()))
            kb, vb = [], []
            for p in range(pages_per_seq[s]):
                kp, vp = blocks_from_export(st, p, g, basis16)
                kb.append((kp, p * page, (p + 1) * page))
                vb.append((vp, p * page, (p + 1) * page))
            tl = tail_lens[s]
            ref[s] = O.chunked_dequant_attention(
                q[s].float().cpu().numpy()[:, None, :], kb, vb, k_arm="lowrank_rtn_channel", v_arm="turboquant_mse_perhead",
                group=group, k_pre_rope=True, rope_cos=cosf, rope_sin=sinf, k_tail=k_tail[s, :, :tl].float().cpu().numpy(),
                v_tail=v_tail[s, :, :tl].float().cpu().numpy(), n_q_groups=G, scale=scale, v_signs=signs.cpu().numpy())[:, 0, :]
        return ref

    K.k2b_decode_static_status()  # readable at any time; before the first static call on a device it reports nothing
    for attempt in range(2):  # two calls in a row on the shared scratch, with different queries
        q = (torch.randn(n_seq, h_kv * G, D, generator=gen) / math.sqrt(D)).half().to(dev)
        ws = K.decode_workspace(g, n_seq, n_pg, dev)
        ref = torch.empty(n_seq, h_kv * G, D, dtype=out_dtype, device=dev)
        K.k2b_decode(pool, q, b16, table, n_pages, n_pg, cos, sin, k_tail, v_tail, tail_len, lut, signs, scale, ws, out=ref)
        out = torch.full((n_seq, h_kv * G, D), float("nan"), dtype=out_dtype, device=dev)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        K.k2b_decode_static(pool, q, b16, table, n_pages, n_pg, cos, sin, k_tail, v_tail, tail_len, lut, signs, scale, out)
        torch.cuda.synchronize()
        if attempt == 1:  # the first call on a device may load the module lazily; from the second on nothing may move
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the static entry point changed the free device memory"
        K.k2b_decode_static_status()  # raises if a bounded wait ran out inside the call
        _tol_check(out.float().cpu().numpy(), ref.float().cpu().numpy(), "static vs workspace entry point")
        _tol_check(out.float().cpu().numpy(), oracle(q), "static entry point vs oracle")

    # a batch whose partial states do not fit the built-in scratch is refused, with both sizes in the message
    big_g = K.k2b_geom(64, 8, page, rank, group, 64, layout=layout)
    big_q = torch.zeros(64, 64 * 8, D, dtype=torch.float16, device=dev)
    with pytest.raises(BmxkError) as ei:
        K.k2b_decode_static(K.K2bPool(big_g, 1, dev), big_q, b16, table, torch.zeros(64, dtype=torch.int32, device=dev), 1,
                            cos, sin, None, None, None, lut, signs, scale,
                            torch.empty(64, 64 * 8, D, dtype=torch.float16, device=dev))
    assert "scratch" in str(ei.value) and str(K.STATIC_SCRATCH_BYTES) in str(ei.value)


def test_static_scratch_on_a_second_device():
    """One process driving two GPUs: the scratch address, the shared-memory opt-in and the SM count are per device."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from bmx_b200 import kernels as K
    from bmx_b200.rope import default_rope_tables

    outs = []
    for idx in (0, 1):
        dev = torch.device("cuda", idx)
        with torch.cuda.device(dev):
            h_kv, G, D, page, rank, group = 2, 4, 128, 128, 32, 64
            gen = torch.Generator().manual_seed(9)
            g = K.k2b_geom(h_kv, G, page, rank, group, h_kv)
            pool = K.K2bPool(g, 3, dev)
            basis = torch.linalg.qr(torch.randn(h_kv, D, rank, generator=gen))[0].reshape(h_kv * D, rank).contiguous()
            k = torch.randn(1, h_kv, 3 * page, D, generator=gen).half().to(dev)
            v = torch.randn(1, h_kv, 3 * page, D, generator=gen).half().to(dev)
            signs, cb = K.hadamard_signs(D, 0).to(dev), torch.tensor(K.GAUSSIAN_CODEBOOK[2], device=dev)
            table = torch.arange(3, dtype=torch.int32, device=dev).view(1, 3)
            K.k2b_append(pool, k, v, basis.to(dev), signs, cb, table.reshape(-1).contiguous(), 3)
            cos, sin = (t.half().to(dev) for t in default_rope_tables(500000.0, D, 1024))
            q = (torch.randn(1, h_kv * G, D, generator=gen) / math.sqrt(D)).half().to(dev)
            out = torch.empty(1, h_kv * G, D, dtype=torch.float32, device=dev)
            K.k2b_decode_static(pool, q, basis.half().to(dev), table, torch.tensor([3], dtype=torch.int32, device=dev), 3, cos, sin,
                                None, None, None, K.v_lut_tensor(K.GAUSSIAN_CODEBOOK[2], dev), signs, 1.0 / math.sqrt(D), out)
            torch.cuda.synchronize()
            K.k2b_decode_static_status()
            outs.append(out.cpu().numpy())
    assert np.all(np.isfinite(outs[1])) and np.array_equal(outs[0], outs[1])
