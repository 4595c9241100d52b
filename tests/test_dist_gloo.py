"""Host-side logic of the multi-GPU partitions, run as two gloo ranks on CPU: page split, head/sequence
shards, the all-gather of partial states and the cross-rank merge formula (no CUDA kernel is called)."""

import math
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from bmx_b200.dist import PART_STRIDE, gather_partials, shard_range, split_pages
from oracle import bmx_oracle as O


def test_partitions_cover_and_balance():
    for n, w in ((1024, 8), (10, 4), (3, 8), (0, 2), (7, 1)):
        parts = split_pages(n, w)
        assert sum(c for _, c in parts) == n and len(parts) == w
        assert max(c for _, c in parts) - min(c for _, c in parts) <= 1
        pos = 0
        for s, c in parts:
            assert s == pos
            pos += c
    assert [shard_range(8, 8, r) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert shard_range(64, 8, 3) == (24, 32)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)  # same data on every rank
        h_kv, G, d, T = 2, 4, 128, 640
        q = (rng.standard_normal((h_kv, G, d)) / math.sqrt(d)).astype(np.float32)
        k = rng.standard_normal((h_kv, T, d)).astype(np.float32)
        v = rng.standard_normal((h_kv, T, d)).astype(np.float32)
        scale = 1.0 / math.sqrt(d)
        first, count = split_pages(T // 128, world)[rank]
        sl = slice(first * 128, (first + count) * 128)
        acc, m, l = O.tail_partial(q, k[:, sl], v[:, sl], scale)
        part = np.zeros((h_kv * G, PART_STRIDE), np.float32)
        part[:, 0] = (m * math.log2(math.e)).reshape(-1)  # the kernels carry maxima in log2 units
        part[:, 1] = l.reshape(-1)
        part[:, 2:] = acc.reshape(-1, d)
        gathered = gather_partials(torch.from_numpy(part)).numpy()
        assert gathered.shape == (world, h_kv * G, PART_STRIDE)
        M = gathered[:, :, 0].max(axis=0)
        w = np.exp2(gathered[:, :, 0] - M[None])
        out = (gathered[:, :, 2:] * w[..., None]).sum(0) / (gathered[:, :, 1] * w).sum(0)[:, None]
        a_full, _, l_full = O.tail_partial(q, k, v, scale)
        ref = (a_full / l_full[..., None]).reshape(-1, d)
        q_out.put((rank, float(np.abs(out - ref).max() / np.abs(ref).max())))
    finally:
        dist.destroy_process_group()


def test_sequence_split_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    qd = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, qd)) for r in range(2)]
    for p in procs:
        p.start()
    res = [qd.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r for r, _ in res) == [0, 1]
    assert all(err < 1e-5 for _, err in res), res
