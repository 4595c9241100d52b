"""Run under torchrun (one rank per GPU): KV heads of one layer split across the ranks while the key basis spans all
heads.  Every rank appends the same tokens for ITS heads (one all-gather for the basis fit, one all-reduce of the partial
projections per flush) and decodes them; the result must equal the heads' slice of a single-GPU state over all heads.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29533 \
        tests/multi_gpu_headshard.py
"""

import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    from bmx_b200 import kernels as K
    from bmx_b200.dist import HeadShardedK2bLayer
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    B, h_kv, G, D, rank_k, page, group, W = 2, 8, 4, 128, 16, 128, 64, 64
    T = 3 * page + W + 20
    gen = torch.Generator(device=dev).manual_seed(7000)  # identical data on every rank
    mix = torch.randn(rank_k, h_kv * D, generator=gen, device=dev)
    coef = torch.randn(B, T, rank_k, generator=gen, device=dev) * torch.arange(1, rank_k + 1, device=dev).float() ** -1.2
    k_pre = (coef @ mix * 0.3 + 0.1 * torch.randn(B, T, h_kv * D, generator=gen, device=dev)).view(B, T, h_kv, D).permute(0, 2, 1, 3).half().contiguous()
    v = torch.randn(B, h_kv, T, D, generator=gen, device=dev).half()
    q = (torch.randn(B, h_kv * G, D, generator=gen, device=dev) / math.sqrt(D)).half()
    cos, sin = default_rope_tables(500000.0, D, T + 256, device=dev)
    k_post = apply_rope(k_pre.float(), cos[:T], sin[:T]).half()

    full = K2bLayerState(K.k2b_geom(h_kv, G, page, rank_k, group, 1), B, T + 256, W, dev, cos.half(), sin.half())
    full.append(k_pre, k_post, v)                       # fits the basis on the first page of all heads
    ref = full.decode(q).float()

    sh = HeadShardedK2bLayer(h_kv, G, rank_k, group, B, T + 256, W, dev, cos.half(), sin.half())
    h0, h1 = sh.h0, sh.h1
    st = sh.state()
    st.append(k_pre[:, h0:h1].contiguous(), k_post[:, h0:h1].contiguous(), v[:, h0:h1].contiguous())
    out = st.decode(q[:, h0 * G:h1 * G].contiguous()).float()
    torch.cuda.synchronize()
    K.check_status(st.workspace)
    same_basis = torch.equal(st.basis_f32, full.basis_f32[h0 * D:h1 * D])
    err = ((out - ref[:, h0 * G:h1 * G]).abs().amax(-1) / ref[:, h0 * G:h1 * G].abs().amax(-1)).max()
    # coefficients: the all-reduce sums the ranks' partial products in another order than one GPU does
    n_pg = st.committed // page
    mine = K.k2b_export_stacks(st.pool, st.page_table[0, :n_pg].contiguous())["us"].float()
    theirs = K.k2b_export_stacks(full.pool, full.page_table[0, :n_pg].contiguous())["us"].float()
    frac = float((mine != theirs).float().mean())
    ulp = float(((mine - theirs).abs() / theirs.abs().clamp_min(1e-6)).max())
    ok = bool(same_basis and float(err) <= 2e-3 and st.committed == full.committed and frac <= 0.05 and ulp <= 2e-3)
    print(f"rank {rank}: heads {h0}..{h1 - 1}, basis equal {same_basis}, worst relative error {float(err):.3e}, "
          f"coefficients differing {frac:.4f} (largest relative step {ulp:.1e})")
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("headshard", "OK" if flag.item() else "FAIL")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
