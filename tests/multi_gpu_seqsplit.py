"""Run under torchrun (one rank per GPU): a single sequence's pages split across ranks, partial states
exchanged (an NCCL all-gather + merge kernel, and the one-kernel peer exchange) and merged, against the same
sequence decoded whole on rank 0; then a step that one rank skips, which must end the others' bounded wait with a
status word and leave the GPUs usable.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29531 \
        tests/multi_gpu_seqsplit.py
"""

import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from bmx_b200 import kernels as K
    from bmx_b200.dist import SequenceSplitDecoder, split_pages
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    h_kv, G, D, rank_k, page, group, W, n_pages = 8, 4, 128, 32, 128, 64, 128, 64
    T = n_pages * page + W
    gen = torch.Generator(device=dev).manual_seed(4000)  # identical data on every rank
    basis = torch.zeros(h_kv * D, rank_k, device=dev)
    for h in range(h_kv):
        Q, _ = torch.linalg.qr(torch.randn(D, rank_k, generator=gen, device=dev))
        basis[h * D:(h + 1) * D] = Q
    k_pre = torch.randn(1, h_kv, T, D, generator=gen, device=dev).half()
    v = torch.randn(1, h_kv, T, D, generator=gen, device=dev).half()
    q = (torch.randn(1, h_kv * G, D, generator=gen, device=dev) / math.sqrt(D)).half()
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)
    k_post = apply_rope(k_pre.float(), cos[:T], sin[:T]).half()
    geom = K.k2b_geom(h_kv, G, page, rank_k, group, h_kv)

    def make_state(first, count, with_window):
        st = K2bLayerState(geom, 1, max(count, 1) * page, W, dev, cos.half(), sin.half())
        st.set_basis(basis)
        if count:
            sl = slice(first * page, (first + count) * page)
            K.k2b_append(st.pool, k_pre[:, :, sl].contiguous(), v[:, :, sl].contiguous(), st.basis_f32, st.signs, st.codebook,
                         st.page_table[0, :count].contiguous(), count)
            st.committed = count * page
            st.n_pages_dev.fill_(count)
        if with_window:
            st.k_win[:, :, :W] = k_post[:, :, n_pages * page:]
            st.v_win[:, :, :W] = v[:, :, n_pages * page:]
            st.tail_len = W
            st.tail_len_dev.fill_(W)
        return st

    first, count = split_pages(n_pages, world)[rank]
    state = make_state(first, count, rank == world - 1)
    whole = make_state(0, n_pages, True) if rank == 0 else None
    ok = True
    for exchange in ("nccl", "p2p"):
        dec = SequenceSplitDecoder(state, first, exchange=exchange)
        for step in range(5):  # several steps: the exchange buffers alternate by step parity
            qs = (q.float() * (1.0 + 0.1 * step)).half()
            out = dec.decode(qs).float()
            torch.cuda.synchronize()
            if dec.peers is not None:
                dec.peers.check()
            if rank == 0:
                ref = whole.decode(qs).float().view(-1, D)
                err = (out - ref).abs().amax(-1) / ref.abs().amax(-1)
                ok = ok and bool((err <= 2e-3).all())
                if step in (0, 4):
                    print(f"seqsplit world={world} {exchange} step {step}: worst relative error vs single-GPU decode {float(err.max()):.3e}")
        if exchange == "p2p":  # the same step replayed from a CUDA graph (the kernel counts its own steps), then eager again
            q_st, out_st = q.clone(), torch.empty(h_kv * G, D, dtype=torch.float32, device=dev)
            graph = dec.capture(q_st, out_st)
            for step in range(4):
                q_st.copy_((q.float() * (1.0 - 0.05 * step)).half())
                dec.replay(graph)
            out = dec.decode(q_st).float()  # host-numbered step after the replays
            torch.cuda.synchronize()
            dec.peers.check()
            if rank == 0:
                ref = whole.decode(q_st).float().view(-1, D)
                e1 = ((out_st - ref).abs().amax(-1) / ref.abs().amax(-1)).max()
                e2 = ((out - ref).abs().amax(-1) / ref.abs().amax(-1)).max()
                ok = ok and float(e1) <= 2e-3 and float(e2) <= 2e-3
                print(f"seqsplit world={world} p2p graph replay / eager after it: {float(e1):.3e} / {float(e2):.3e}")
        dec.close()
    # ---- one rank skips a step: the others' wait must run out (1 ms limit here), say who was missing, and return ----
    from bmx_b200.dist import PeerExchange

    px = PeerExchange(h_kv * G, dev)
    px.WAIT_LIMIT_CYCLES = 2_000_000
    part = torch.zeros(h_kv * G, 130, device=dev)
    part[:, 1] = 1.0
    px.merge(part)
    torch.cuda.synchronize()
    px.check()  # a complete step first
    if rank != world - 1:
        px.merge(part)  # the last rank never makes this call
        torch.cuda.synchronize()
        st = px.status.cpu().tolist()
        gave_up = st[0] == 1 and st[2] == 32 + (world - 1)
        ok = ok and gave_up
        if rank == 0:
            print(f"skipped step: status {st[:3]} -> {'the wait named the missing rank' if gave_up else 'UNEXPECTED'}")
        # the context is still usable
        ok = ok and bool(torch.isfinite(state.decode(q, partial_out=None).float()).all())
    px.close()
    if rank == 0:
        print("seqsplit", "OK" if ok else "FAIL")
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    ok = bool(flag.item())
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
