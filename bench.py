#!/usr/bin/env python
"""Benchmark of the packed k2b KV-cache decode path (one attention layer-step).

Workload (synthetic, seeded): Llama-3.1-8B head shape (32 query heads, 8 KV heads, head dim 128),
B = 8 sequences, 32768 committed tokens + a 128-token fp16 window per sequence; keys pre-RoPE with
a per-head rank-32 basis and a 3-bit residual, values Hadamard + 2-bit Lloyd codes, RoPE theta
500000 applied at read.  One step = one decode call over the whole batch (two kernel launches).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 (launched by torchrun, one rank per GPU) every rank holds its own B = 8 batch: KV heads
and sequences are independent, so the path shards with no collective ("weak" scaling); the time is
the maximum over ranks.  The same line carries, under `configs`, device timings of the path's other
configurations: the RTN cache (B = 1, T = 4096), quantize-on-append (B = 16), the K4 spectral cache
(B = 64 over all ranks) and one 131072-token sequence split across the ranks with one NCCL all-gather
per step.  `--impl reference` times the CPU restatement of the reference's chunked dequant-attention
(oracle/) on the host cores over a bounded, named sample of the same workload.
Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

H_KV, G, D, RANK, PAGE, GROUP, WINDOW = 8, 4, 128, 32, 128, 64, 128
BATCH, CTX = 8, 32768
BYTES_PER_UNIT = 166  # per (token, kv head): coefficients 64 + residual nibbles 64 + scales 4 + value codes 32 + norm 2
ROPE_THETA = 500000.0
# dram__bytes_read.sum + dram__bytes_write.sum of one k2b_decode_t5_kernel launch from an ncu capture at 16384 tokens
# (174.68 + 4.66 MB), scaled by 2 to this workload's 32768 tokens: the kernel streams every page once, so traffic grows
# in proportion to the tokens.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2 * (174.68e6 + 4.66e6)


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index: int):
        self.index, self.rows, self.proc, self.windows = index, [], None, []

    def mark(self, t0: float, t1: float) -> None:
        """[t0, t1] (time.perf_counter) was spent under the measured load: only samples taken then are summarised."""
        self.windows.append((t0, t1))

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")] + [time.perf_counter()])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        # a sample describes the ~50 ms before it was printed: keep those printed inside a load window or just after it
        rows = [r for r in self.rows if not self.windows or any(t0 <= r[-1] <= t1 + 0.06 for t0, t1 in self.windows)]
        mhz = sorted(int(r[0]) for r in rows if r and str(r[0]).isdigit())
        mx = [int(r[1]) for r in rows if len(r) > 1 and str(r[1]).isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in rows)]
        watts = []
        for r in rows:
            try:
                watts.append(float(r[6]))
            except (IndexError, ValueError):
                pass
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(mhz), "power_w_max": max(watts) if watts else None}


# ------------------------------------------------------------------------------------------------
# synthetic workload
# ------------------------------------------------------------------------------------------------

def make_basis(gen, device):
    import torch

    basis = torch.zeros(H_KV * D, RANK, device=device)
    for h in range(H_KV):
        Q, R = torch.linalg.qr(torch.randn(D, RANK, generator=gen, device=device))
        basis[h * D:(h + 1) * D] = Q * torch.sign(torch.diagonal(R))
    return basis


def make_kv(gen, basis, n_seq, T, device):
    """Pre-RoPE keys = per-head low-rank signal (spectrum i^-1.5) + 0.1 N(0,1); values N(0,1)."""
    import torch

    decay = torch.arange(1, RANK + 1, device=device).float() ** -1.5
    coef = torch.randn(n_seq, H_KV, T, RANK, generator=gen, device=device) * decay
    k = torch.einsum("bhtr,hcr->bhtc", coef, basis.view(H_KV, D, RANK))
    k = (k + 0.1 * torch.randn(n_seq, H_KV, T, D, generator=gen, device=device)).half()
    v = torch.randn(n_seq, H_KV, T, D, generator=gen, device=device).half()
    return k, v


def build_state(device, seed, batch=BATCH, ctx=CTX):
    """A K2bLayerState holding `ctx` committed tokens + a full window, filled through the append kernel."""
    import torch

    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables

    gen = torch.Generator(device=device).manual_seed(seed)
    total = ctx + WINDOW
    cos, sin = default_rope_tables(ROPE_THETA, D, total + 4096, device=device)
    geom = K.k2b_geom(H_KV, G, PAGE, RANK, GROUP, H_KV)
    state = K2bLayerState(geom, batch, total + 4096, WINDOW, device, cos.half(), sin.half())
    basis = make_basis(gen, device)
    state.set_basis(basis)
    # one sequence at a time through a scratch state keeps the transient fp16 K/V small
    for b in range(batch):
        k_pre, v = make_kv(gen, basis, 1, total, device)
        k_post = apply_rope(k_pre.float(), cos[:total], sin[:total]).half()
        n_pg = ctx // PAGE
        slots = state.page_table[b, :n_pg].contiguous()
        K.k2b_append(state.pool, k_pre, v, state.basis_f32, state.signs, state.codebook, slots, n_pg)
        state.k_win[b, :, :WINDOW] = k_post[0, :, ctx:]
        state.v_win[b, :, :WINDOW] = v[0, :, ctx:]
        state.k_pre_win[b, :, :WINDOW] = k_pre[0, :, ctx:]
    state.committed, state.tail_len = ctx, WINDOW
    state.n_pages_dev.fill_(ctx // PAGE)
    state.tail_len_dev.fill_(WINDOW)
    q = (torch.randn(batch, H_KV * G, D, generator=gen, device=device) / math.sqrt(D)).half()
    return state, q, gen, basis, (cos, sin)


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle's chunked dequant-attention over a bounded sample of the same workload
# ------------------------------------------------------------------------------------------------

def _host_cores() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


class CpuReference:
    """The CPU arm: oracle.chunked_dequant_attention (a numpy restatement of bmx's chunked dequant-attention, all BLAS
    threads) over `n_pages` pages of ONE sequence of the workload (8 KV heads, 32 query heads), pages quantized by the
    oracle codec.  A step attends over the whole sample once; the metric is a rate (packed bytes consumed per second),
    so it does not depend on the sample size, and the sample is named in the output."""

    def __init__(self, n_pages: int, seed: int = 2000):
        import numpy as np
        import torch  # only for the seeded sign vector, as the reference draws it

        from oracle import bmx_oracle as O

        self.O, self.n_pages = O, n_pages
        rng = np.random.default_rng(seed)
        C = H_KV * D
        basis = np.zeros((C, H_KV * RANK), np.float32)  # block-diagonal: one rank-32 basis per head
        for h in range(H_KV):
            Qm, _ = np.linalg.qr(rng.standard_normal((D, RANK)).astype(np.float32))
            basis[h * D:(h + 1) * D, h * RANK:(h + 1) * RANK] = Qm
        g = torch.Generator().manual_seed(0)
        self.signs = (torch.randint(0, 2, (D,), generator=g) * 2 - 1).numpy().astype(np.float32)
        decay = (np.arange(1, RANK + 1, dtype=np.float32) ** -1.5)
        cos, sin = O.default_rope_tables(ROPE_THETA, D, n_pages * PAGE)
        self.cos16, self.sin16 = cos.astype(np.float16).astype(np.float32), sin.astype(np.float16).astype(np.float32)
        self.q = (rng.standard_normal((H_KV * G, 1, D)) / math.sqrt(D)).astype(np.float32)
        self.kb, self.vb = [], []
        for p in range(n_pages):
            coef = rng.standard_normal((PAGE, H_KV * RANK)).astype(np.float32) * np.tile(decay, H_KV)
            Mk = (coef @ basis.T + 0.1 * rng.standard_normal((PAGE, C)).astype(np.float32)).astype(np.float16).astype(np.float32)
            Mv = rng.standard_normal((PAGE, C)).astype(np.float16).astype(np.float32)
            kp, _ = O.quantize_packed("lowrank_rtn_channel", Mk, bits=3, group=GROUP, rank=RANK, svd_factors=(Mk @ basis, basis))
            vp, _ = O.quantize_packed("turboquant_mse_perhead", Mv, bits=2, h_heads=H_KV, signs=self.signs)
            self.kb.append((kp, p * PAGE, (p + 1) * PAGE))
            self.vb.append((vp, p * PAGE, (p + 1) * PAGE))
        self.units = n_pages * PAGE * H_KV

    def step(self) -> float:
        t0 = time.perf_counter()
        self.O.chunked_dequant_attention(self.q, self.kb, self.vb, k_arm="lowrank_rtn_channel", v_arm="turboquant_mse_perhead",
                                         group=GROUP, k_pre_rope=True, rope_cos=self.cos16, rope_sin=self.sin16, k_tail=None,
                                         v_tail=None, n_q_groups=G, scale=1.0 / math.sqrt(D), v_signs=self.signs)
        return time.perf_counter() - t0

    def sample(self) -> str:
        return (f"{self.n_pages} pages x {PAGE} tokens x {H_KV} kv heads of one sequence ({self.units} of {BATCH * H_KV * CTX} units of "
                f"the workload), numpy restatement of bmx chunked_dequant_attention")


def cpu_pages_for(total_budget_s: float, n_steps: int) -> int:
    """Pages per step such that n_steps steps take about total_budget_s: a whole sequence (256 pages) if that fits."""
    probe = CpuReference(8)
    probe.step()
    per_page = probe.step() / 8
    return int(max(8, min(CTX // PAGE, total_budget_s / max(n_steps, 1) / max(per_page, 1e-5))))


def cpu_baseline_leg(budget_s: float = 12.0):
    """cpu_baseline of the GPU arm's line: one warm-up step and up to three timed steps over a bounded sample."""
    n = cpu_pages_for(budget_s, 4)
    ref = CpuReference(n)
    ref.step()
    times = [ref.step() for _ in range(3)]
    dt = sum(times) / len(times)
    return {"value": ref.units * BYTES_PER_UNIT / dt / 1e9, "unit": "GB/s", "cores": _host_cores(), "kind": "port",
            "sample": ref.sample(), "ms_per_sample_step": dt * 1e3,
            "us_per_layer_step_extrapolated": dt / ref.units * (BATCH * H_KV * CTX) * 1e6}


def run_reference(args, rank):
    """`--impl reference`: W warm-up and exactly K timed steps of the CPU arm on rank 0; every step attends over the
    sample named in config.workload (one whole sequence of the workload when K steps of it fit in about two minutes)."""
    if rank != 0:
        return
    warm = max(args.warmup, 1)
    n = cpu_pages_for(120.0, args.steps + warm)
    ref = CpuReference(n)
    for _ in range(warm):
        ref.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ref.step()
    dt = (time.perf_counter() - t0) / args.steps
    gbs = ref.units * BYTES_PER_UNIT / dt / 1e9
    cfg = workload_config(args.gpus)
    cfg["workload"] = ("CPU arm: " + ref.sample() + "; same geometry and distributions as the GPU arm's workload (" + cfg["workload"] + ")")
    cfg["sample_pages_per_step"], cfg["sample_units_per_step"] = n, ref.units
    line = {
        "impl": "reference", "metric": "k2b_decode_effective_GBps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "us_per_layer_step_extrapolated": dt / ref.units * (BATCH * H_KV * CTX) * 1e6,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": _host_cores(), "kind": "port", "sample": ref.sample()},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "k2b packed-cache decode, 1 layer-step: Llama-3.1-8B heads (32 q / 8 kv, d=128), B=8 per GPU, "
                        "T=32768 committed + 128-token fp16 window, K rank-32 per-head basis + 3-bit residual (group 64), "
                        "V Hadamard + 2-bit Lloyd, RoPE theta 5e5 at read, 128-token pages",
            "batch_per_gpu": BATCH, "context": CTX, "window": WINDOW, "page": PAGE, "rank": RANK,
            "bytes_per_token_head": BYTES_PER_UNIT, "parallelism": f"kv-head/batch shards x{n_gpus}, no collective",
            "l2": "packed pages read per step (348 MB per GPU) exceed the 126 MB L2; no explicit flush"}


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------

def run_ours(args, rank, world, local_rank):
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the bmxk kernels have no CPU path")
    import torch.distributed as dist

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        from datetime import timedelta

        # a rank that fails leaves the others in a collective: give up after two minutes, not the default ten
        dist.init_process_group("nccl", device_id=device, timeout=timedelta(seconds=120))
    clocks = ClockSampler(local_rank).__enter__()  # started before the workload is built: nvidia-smi needs a moment to print its first line
    state, q, gen, basis, (cos, sin) = build_state(device, seed=2000 + rank, ctx=args.ctx)
    from bmx_b200 import kernels as K

    out = torch.empty(BATCH, H_KV * G, D, dtype=torch.float16, device=device)
    units = BATCH * H_KV * args.ctx
    algo_bytes = units * BYTES_PER_UNIT

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Clock samples: nvidia-smi prints one line per 50 ms, so the timed steps (a few tens of ms) would catch one at best.
    # The same decode call therefore keeps running for 0.35 s after the timed steps and the per-kernel loop, and the
    # samples printed between the first warm-up step and the end of that tail are the ones summarised.  The warm-up
    # BEFORE the timed steps is the W steps asked for and no more (on one box the same steps ran ~4 % slower after a long
    # pre-heating loop, with the sampled SM clock unchanged; on another they did not).
    t_load = time.perf_counter()
    for _ in range(max(args.warmup, 3)):
        state.decode(q, out=out)
    torch.cuda.synchronize()
    K.check_status(state.workspace)

    # ---- device-resident steps: K decode calls (the user's call: both kernels) back to back ----
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        state.decode(q, out=out)
    e1.record()
    barrier()
    total_ms = e0.elapsed_time(e1)
    # ---- the same steps once more with the two kernels launched apart and events between them on the launching
    #      stream: the duration of the dominant kernel for the roofline (phase 1 = page-streaming kernel, phase 2 =
    #      merge kernel; launched apart, the merge kernel does not overlap the other's drain) ----
    n_k = min(args.steps, 100)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_k)]
    for i in range(n_k):
        ev[i][0].record()
        state.decode(q, out=out, phases=1)
        ev[i][1].record()
        state.decode(q, out=out, phases=2)
        ev[i][2].record()
    torch.cuda.synchronize()
    main_ms = sum(e[0].elapsed_time(e[1]) for e in ev) / n_k
    merge_ms = sum(e[1].elapsed_time(e[2]) for e in ev) / n_k
    K.check_status(state.workspace)
    n_tail = 0
    while time.perf_counter() - t_load < 0.35:
        state.decode(q, out=out)
        n_tail += 1
        if n_tail % 16 == 0:
            torch.cuda.synchronize()
    torch.cuda.synchronize()
    clocks.mark(t_load, time.perf_counter())

    # ---- the step's own output checked against the CPU oracle on the same stored pages, for one (sequence, head) at
    #      the full context (rank 0 only; outside every timed region) ----
    selfcheck = None
    if rank == 0:
        selfcheck = oracle_check_one_head(state, q, seq=0, head=min(3, H_KV - 1))
        assert selfcheck["max_rel_err"] <= 2e-3, f"decode output off the oracle: {selfcheck}"

    # ---- end to end through the layer-state API with host buffers: per step the new token's K/V and
    #      the query come from pinned host memory, the attention output goes back to the host ----
    # DecodeStepGraph: one pinned staging buffer [q | k_post | v | k_pre] in, the attention output out; the copies, the
    # window append and the two decode kernels replay as one CUDA graph; the step on which the flush schedule commits
    # a page per sequence (one in 128) replays a graph of its own (ingest, slot lookup, page quantizer, window shift, decode).
    # 160 timed steps after a warm-up that crosses one commit: the timed region holds exactly one such step.
    n_e2e = 160
    from bmx_b200.engine import DecodeStepGraph

    nq, nk = BATCH * H_KV * G * D, BATCH * H_KV * D
    hin = torch.empty(nq + 3 * nk, dtype=torch.float16).pin_memory()
    hin[:nq].copy_(q.cpu().reshape(-1))
    hin[nq:].copy_((0.3 * torch.randn(3 * nk)).half())
    hout = torch.empty(BATCH, H_KV * G, D, dtype=torch.float16).pin_memory()
    stepper = DecodeStepGraph(state, hin, hout)
    h2d = hin.numel() * 2  # q, the new token's post-RoPE key, value and pre-RoPE key
    d2h = hout.numel() * 2

    def e2e_step():
        stepper.step()
        torch.cuda.current_stream().synchronize()

    t_load = time.perf_counter()
    for _ in range(PAGE + 4):  # warm-up across one page commit: both graphs of the stepper (plain step, flush step) exist afterwards
        e2e_step()
    barrier()
    committed_before = state.committed
    step_wall = []
    t0 = time.perf_counter()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(n_e2e):
        t1 = time.perf_counter()
        e2e_step()
        step_wall.append(time.perf_counter() - t1)
    g1.record()
    torch.cuda.synchronize()
    e2e_ms = max(g0.elapsed_time(g1), (time.perf_counter() - t0) * 1e3) / n_e2e
    flush_steps = (state.committed - committed_before) // PAGE
    flush_us = max(step_wall) * 1e6
    plain_us = sorted(step_wall)[len(step_wall) // 2] * 1e6
    K.check_status(state.workspace)
    clocks.mark(t_load, time.perf_counter())
    time.sleep(0.06)  # the sample that covers the end of the last window
    clocks.__exit__(None, None, None)

    mine = torch.tensor([total_ms / args.steps, main_ms, merge_ms, e2e_ms], dtype=torch.float64, device=device)
    per_rank = mine.clone().unsqueeze(0)
    if world > 1:
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        per_rank = torch.stack(gathered)
    ms_per_step, main_ms, merge_ms, e2e_ms = per_rank.max(0).values.tolist()

    # ---- the other configurations of the path (device timings with CUDA events; each builds and frees its own state) ----
    del stepper
    state = None
    torch.cuda.empty_cache()
    extra = {}
    if rank == 0:
        extra["rtn_b1_t4096"] = config_rtn(device)
        extra["append_b16"] = config_append(device)
        extra["prefill_b1_t16384"] = config_prefill(device)
        extra["latency_b1"] = config_latency_b1(device)
    extra_all = {"spectral_b64_t16384": config_spectral(device, rank, world, dist if world > 1 else None),
                 "seq_split_t131072": config_seq_split(device, rank, world, dist if world > 1 else None)}

    if rank == 0:
        extra.update(extra_all)
        peak, peak_kind = measured_peak_gbs()
        achieved = algo_bytes / (main_ms * 1e-3) / 1e9
        cpu = cpu_baseline_leg(10.0) if world == 1 else None
        cols = ("ms_per_step", "kernel_ms", "merge_kernel_ms", "e2e_ms")
        line = {
            "metric": "k2b_decode_effective_GBps", "value": world * algo_bytes / (ms_per_step * 1e-3) / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "us_per_layer_step": ms_per_step * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": dict(workload_config(world), context=args.ctx),
            "frac_of_8TBps": world * algo_bytes / (ms_per_step * 1e-3) / 1e9 / (8000.0 * world),
            "roofline": {"bound": "hbm", "kernel": "k2b_decode_t5_kernel<32,4>", "achieved": achieved, "peak": peak,
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind})", "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH * args.ctx / CTX, "algorithmic_bytes": algo_bytes,
                         "kernel_us": main_ms * 1e3, "merge_kernel_us": merge_ms * 1e3},
            "cpu_baseline": cpu,
            "e2e": {"value": world * algo_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "us_per_layer_step": e2e_ms * 1e3,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": n_e2e, "flush_steps_in_region": int(flush_steps),
                    "us_flush_step": flush_us, "us_median_step": plain_us},
            "per_rank": [dict(zip(cols, row)) for row in per_rank.tolist()],
            "oracle_check": selfcheck,
            "configs": extra,
            "gpu_launches": 2 * args.steps,
            "clocks": clocks.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def oracle_check_one_head(state, q, seq: int, head: int) -> dict:
    """Decodes once into a float32 buffer and compares (sequence, head) with the CPU oracle's chunked dequant-attention
    over the pages as stored (exported in bmx's layout) plus the fp16 window.  The oracle is the checker here."""
    import numpy as np
    import torch

    from bmx_b200 import kernels as K
    from oracle import bmx_oracle as O

    g = state.geom
    out = torch.empty(state.batch, g.h_kv * g.n_q_groups, D, dtype=torch.float32, device=state.device)
    state.decode(q, out=out)
    torch.cuda.synchronize()
    n_pg, tl = state.committed // PAGE, state.tail_len
    st = {a: t.cpu().numpy() for a, t in K.k2b_export_stacks(state.pool, state.page_table[seq, :n_pg].contiguous()).items()}
    basis16 = state.basis_f16[head * D:(head + 1) * D].float().cpu().numpy()
    signs = state.signs.cpu().numpy()
    kb, vb = [], []
    for p in range(n_pg):
        kp = {"Us": st["us"][p, head].astype(np.float32), "V": basis16,
              "res_Q_int": O.unpack_signed_codes(st["res_int_packed"][p][head * D:(head + 1) * D], g.kbits, PAGE),
              "res_scale": st["res_scale"][p][head * D:(head + 1) * D].astype(np.float32)[..., None]}
        idx = O.unpack_codes(st["v_idx_packed"][p], 2, g.h_kv * D)[:, head * D:(head + 1) * D]
        vp = {"indices": idx, "norms": st["v_norm"][p][:, head:head + 1].astype(np.float32), "bits": 2, "h": 1}
        kb.append((kp, p * PAGE, (p + 1) * PAGE))
        vb.append((vp, p * PAGE, (p + 1) * PAGE))
    cos, sin = state.rope_cos.float().cpu().numpy(), state.rope_sin.float().cpu().numpy()
    qh = q[seq, head * g.n_q_groups:(head + 1) * g.n_q_groups].float().cpu().numpy()[:, None, :]
    ref = O.chunked_dequant_attention(qh, kb, vb, k_arm="lowrank_rtn_channel", v_arm="turboquant_mse_perhead", group=g.group,
                                      k_pre_rope=True, rope_cos=cos, rope_sin=sin,
                                      k_tail=state.k_win[seq, head:head + 1, :tl].float().cpu().numpy(),
                                      v_tail=state.v_win[seq, head:head + 1, :tl].float().cpu().numpy(), n_q_groups=g.n_q_groups,
                                      scale=state.sm_scale, v_signs=signs)[:, 0, :]
    got = out[seq, head * g.n_q_groups:(head + 1) * g.n_q_groups].cpu().numpy()
    err = np.abs(got - ref).max(axis=-1) / np.abs(ref).max(axis=-1)
    return {"sequence": seq, "kv_head": head, "tokens": state.committed + tl, "max_rel_err": float(err.max()), "bound": 2e-3}


def _event_us(fn, n: int, warm: int = 3) -> float:
    import torch

    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / n


def config_rtn(device) -> dict:
    """Benchmark configuration 1 (plain RTN cache), B = 1, 4096 committed tokens + a 128-token fp16 window; keys rtn_channel 4 bits,
    values rtn_token 2 bits, groups of 32; K ~ N(0,1) with 4 channels per head x 8.  4.2 MB per step: the step is bound by
    launch latency, so it is timed both as plain launches and replayed from a CUDA graph."""
    import torch

    from bmx_b200 import kernels as K
    from bmx_b200.engine import RtnLayerState

    T, W = 4096, 128
    gen = torch.Generator(device=device).manual_seed(1000)
    geom = K.rtn_geom(H_KV, G, PAGE, "rtn_channel", 32, 32, 4, 2)
    st = RtnLayerState(geom, 1, T + 2 * PAGE, W, device)
    k = torch.randn(1, H_KV, T + W, D, generator=gen, device=device)
    k[..., :4] *= 8.0
    v = torch.randn(1, H_KV, T + W, D, generator=gen, device=device)
    st.append(None, k.half(), v.half())
    assert st.committed == T and st.tail_len == W
    q = (torch.randn(1, H_KV * G, D, generator=gen, device=device) / math.sqrt(D)).half()
    out = torch.empty(1, H_KV * G, D, dtype=torch.float16, device=device)
    eager_us = _event_us(lambda: st.decode(q, out=out), 200)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        st.decode(q, out=out)
    graph_us = _event_us(graph.replay, 500)
    K.check_status(st.workspace)
    algo = T * H_KV * 112 + W * H_KV * 512  # codes 64 + 32, fp16 scales 8 + 8 per (token, head); the window is fp16 K and V
    peak, _ = measured_peak_gbs()
    return {"workload": "RTN packed-cache decode: B=1, T=4096 + 128-token window, K rtn_channel 4b / V rtn_token 2b, group 32",
            "us_per_layer_step": eager_us, "us_per_layer_step_graph": graph_us, "algorithmic_bytes": algo,
            "roofline": {"bound": "launch latency (4.2 MB of traffic: 0.64 us at the HBM peak)", "achieved": algo / graph_us / 1e3,
                         "peak": peak, "unit": "GB/s", "frac": algo / graph_us / 1e3 / peak}, "gpu_launches_per_step": 2}


def config_append(device, B: int = 16) -> dict:
    """Benchmark configuration 3: quantize-on-append of the k2b recipe, B = 16, bf16 sources, one layer (the 32 layers of the config
    repeat it).  Bulk: the 16384-token prefix of all sequences in one call (128 pages x 16 sequences x 8 heads).  Streaming:
    single-token steps on top of it, 127 of every 128 move one token into the fp16 window, the 128th commits a page per
    sequence.  Bytes per (page, head): read 2 x 128 x 128 x 2 (key and value sources), write 13056 + 8192."""
    import torch

    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import default_rope_tables

    T0, W = 16384, 128
    gen = torch.Generator(device=device).manual_seed(3000)
    basis = make_basis(gen, device)
    cos, sin = default_rope_tables(ROPE_THETA, D, T0 + 4096, device=device)
    out = {}
    total = T0 + W + 2 * PAGE + 8
    k_pre = torch.empty(B, H_KV, total, D, dtype=torch.bfloat16, device=device)
    v = torch.empty_like(k_pre)
    for b in range(B):
        kb_, vb_ = make_kv(gen, basis, 1, total, device)
        k_pre[b], v[b] = kb_[0].bfloat16(), vb_[0].bfloat16()
    peak, _ = measured_peak_gbs()
    for page in (128, 64):
        geom = K.k2b_geom(H_KV, G, page, RANK, GROUP, H_KV)
        n_pg = T0 // page
        pool = K.K2bPool(geom, B * n_pg, device)
        slots = torch.arange(B * n_pg, dtype=torch.int32, device=device)
        signs, cb = K.hadamard_signs(D, 0).to(device), torch.tensor(K.GAUSSIAN_CODEBOOK[2], device=device)
        us = _event_us(lambda: K.k2b_append(pool, k_pre, v, basis, signs, cb, slots, n_pg), 3, warm=1)
        items = B * n_pg * H_KV
        nbytes = items * (2 * page * D * 2 + K.page_block_bytes(geom) + K.coef_block_bytes(geom))
        out[f"bulk_prefix_page{page}"] = {"us": us, "pages_per_s": B * n_pg / us * 1e6, "page_heads_per_s": items / us * 1e6,
                                          "GBps": nbytes / us / 1e3, "frac_of_hbm_peak": nbytes / us / 1e3 / peak,
                                          "bytes": nbytes, "gpu_launches": 1}
        del pool
    geom = K.k2b_geom(H_KV, G, PAGE, RANK, GROUP, H_KV)
    st = K2bLayerState(geom, B, T0 + 4096, W, device, cos.half(), sin.half())
    st.set_basis(basis)
    n0 = T0 + W
    st.append(k_pre[:, :, :n0], k_pre[:, :, :n0], v[:, :, :n0])  # the post-RoPE window keys do not matter for timing
    assert st.committed == T0 and st.tail_len == W
    plain, flush = [], []
    e = [torch.cuda.Event(enable_timing=True) for _ in range(2 * PAGE + 1)]
    e[0].record()
    for i in range(2 * PAGE):
        t = n0 + i
        st.append(k_pre[:, :, t:t + 1], k_pre[:, :, t:t + 1], v[:, :, t:t + 1])
        e[i + 1].record()
    torch.cuda.synchronize()
    committed = T0
    from bmx_b200.schedule import compute_flush_schedule
    for i in range(2 * PAGE):
        new_c = compute_flush_schedule(n0 + i + 1, W, PAGE)
        (flush if new_c > committed else plain).append(e[i].elapsed_time(e[i + 1]) * 1e3)
        committed = max(committed, new_c)
    assert st.committed == T0 + 2 * PAGE and len(flush) == 2
    step_bytes = B * H_KV * (2 * PAGE * D * 2 + K.page_block_bytes(geom) + K.coef_block_bytes(geom))
    out["streaming_page128"] = {"us_non_flush_step": sorted(plain)[len(plain) // 2], "us_flush_step": sum(flush) / len(flush),
                                "flush_every_steps": PAGE, "bytes_per_flush_step": step_bytes,
                                "us_per_token_all_32_layers": 32 * (sum(plain) + sum(flush)) / (len(plain) + len(flush)),
                                "note": "host-launched steps (torch ops + kernel launches on one stream), one layer"}
    # the same steps as the product runs them: append + decode replayed as CUDA graphs from pinned host buffers (one graph
    # for a plain step, one for a step that commits a page per sequence); the difference of the two is what a commit costs
    from bmx_b200.engine import DecodeStepGraph

    nq, nk = B * H_KV * G * D, B * H_KV * D
    hin = (0.3 * torch.randn(nq + 3 * nk)).half().pin_memory()
    hout = torch.empty(B, H_KV * G, D, dtype=torch.float16).pin_memory()
    stepper = DecodeStepGraph(st, hin, hout)
    walls = []
    for i in range(3 * PAGE):
        t0 = time.perf_counter()
        c0 = st.committed
        stepper.step()
        torch.cuda.current_stream().synchronize()
        walls.append((time.perf_counter() - t0, st.committed > c0))
    K.check_status(st.workspace)
    plain_g = sorted(w for w, f in walls[PAGE + 8:] if not f)
    flush_g = [w for w, f in walls[PAGE + 8:] if f]   # the first commit captured the flush graph: these are replays
    out["graph_steps_from_host_buffers"] = {"us_plain_step": plain_g[len(plain_g) // 2] * 1e6, "us_flush_step": sum(flush_g) / max(1, len(flush_g)) * 1e6,
                                            "flush_steps": len(flush_g), "flush_graph_replays": stepper.flush_replays,
                                            "note": "append + decode of this state (B=16, 16k context) per step, host-synchronised"}
    out["workload"] = "k2b quantize-on-append, B=16, bf16 sources, 16384-token prefix then single-token steps, 128-token window"
    return out


def config_seq_split(device, rank, world, dist) -> dict:
    """Benchmark configuration 4: one sequence of 131072 committed tokens (32 q / 8 kv heads, d 128, k2b recipe), its pages split
    across the ranks; every rank decodes its part into an un-normalised state (max, sum, accumulator), ONE all-gather of
    (32 x 130) floats per rank, then the merge.  Rank 0 also holds the whole sequence and checks the merged output against
    its own single-GPU decode (2e-3).  At one GPU this is just the single-GPU long-context step."""
    import torch

    from bmx_b200 import kernels as K
    from bmx_b200.dist import SequenceSplitDecoder, split_pages
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables

    T, W = 131072, 128
    n_pg = T // PAGE
    gen = torch.Generator(device=device).manual_seed(4000)  # the same sequence on every rank
    basis = make_basis(gen, device)
    cos, sin = default_rope_tables(ROPE_THETA, D, T + 4096, device=device)
    geom = K.k2b_geom(H_KV, G, PAGE, RANK, GROUP, H_KV)
    k_pre, v = make_kv(gen, basis, 1, T + W, device)
    q = (torch.randn(1, H_KV * G, D, generator=gen, device=device) / math.sqrt(D)).half()
    first, count = split_pages(n_pg, world)[rank]
    last = rank == world - 1
    st = K2bLayerState(geom, 1, count * PAGE + 2 * PAGE, W, device, cos.half(), sin.half())
    st.set_basis(basis)
    slots = st.page_table[0, :count].contiguous()
    lo = first * PAGE
    K.k2b_append(st.pool, k_pre[:, :, lo:lo + count * PAGE], v[:, :, lo:lo + count * PAGE], st.basis_f32, st.signs, st.codebook, slots, count)
    st.committed = count * PAGE
    st.n_pages_dev.fill_(count)
    if last:
        k_post = apply_rope(k_pre[:, :, T:].float(), cos[T:T + W], sin[T:T + W]).half()
        st.k_win[:, :, :W], st.v_win[:, :, :W], st.k_pre_win[:, :, :W] = k_post, v[:, :, T:], k_pre[:, :, T:]
        st.tail_len = W
        st.tail_len_dev.fill_(W)
    out = torch.empty(H_KV * G, D, dtype=torch.float32, device=device)
    res = {"workload": "k2b decode, one sequence of 131072 tokens + 128-token window, pages split across the ranks, one exchange "
                       "of (32 x 130) floats per rank, merge on every rank", "pages_per_rank": count}
    if world == 1:
        o1 = torch.empty(1, H_KV * G, D, dtype=torch.float32, device=device)
        step_us = _event_us(lambda: st.decode(q, out=o1), 100)
        kern_us = _event_us(lambda: st.decode(q, out=o1, phases=1), 100)
        K.check_status(st.workspace)
        algo = T * H_KV * BYTES_PER_UNIT
        peak, _ = measured_peak_gbs()
        res.update(us_per_layer_step=step_us, kernel_us=kern_us, achieved_GBps=algo / kern_us / 1e3, frac_of_hbm_peak=algo / kern_us / 1e3 / peak,
                   algorithmic_bytes=algo, collective=None)
        return res
    dec = SequenceSplitDecoder(st, first)
    step_us = _event_us(lambda: dec.decode(q, out=out), 100)
    kern_us = _event_us(lambda: st.decode(q, partial_out=dec.part, pos_offset=first * PAGE, phases=1), 100)
    K.check_status(st.workspace)
    # the same step with the one-kernel peer exchange instead of the all-gather + merge kernel (its set-up raises on every
    # rank together if CUDA IPC is not available between the ranks; the NCCL figures stand in then)
    out_p, p2p_error = torch.empty_like(out), None
    try:
        dec_p = SequenceSplitDecoder(st, first, exchange="p2p")
    except RuntimeError as e:
        dec_p, p2p_error, p2p_us, p2p_graph_us = None, str(e), step_us, step_us
        out_p.copy_(out)
    if dec_p is not None:
        dist.barrier()
        p2p_us = _event_us(lambda: dec_p.decode(q, out=out_p), 100)
        dec_p.peers.check()
        graph = dec_p.capture(q, out_p)  # the three launches of a step replayed as one graph
        dist.barrier()
        p2p_graph_us = _event_us(lambda: dec_p.replay(graph), 100)
        dec_p.peers.check()
        dec_p.close()
    t = torch.tensor([step_us, kern_us, p2p_us, p2p_graph_us], dtype=torch.float64, device=device)
    allt = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(allt, t)
    allt = torch.stack(allt)
    # rank 0 decodes the whole sequence by itself and compares
    max_rel = None
    if rank == 0:
        full = K2bLayerState(geom, 1, T + 2 * PAGE, W, device, cos.half(), sin.half())
        full.set_basis(basis)
        K.k2b_append(full.pool, k_pre[:, :, :T], v[:, :, :T], full.basis_f32, full.signs, full.codebook,
                     full.page_table[0, :n_pg].contiguous(), n_pg)
        full.committed = T
        full.n_pages_dev.fill_(n_pg)
        k_post = apply_rope(k_pre[:, :, T:].float(), cos[T:T + W], sin[T:T + W]).half()
        full.k_win[:, :, :W], full.v_win[:, :, :W], full.k_pre_win[:, :, :W] = k_post, v[:, :, T:], k_pre[:, :, T:]
        full.tail_len = W
        full.tail_len_dev.fill_(W)
        o1 = torch.empty(1, H_KV * G, D, dtype=torch.float32, device=device)
        full.decode(q, out=o1)   # `out` still holds the last timed step's merged result: no rank-0-only collective here
        torch.cuda.synchronize()
        err = (out - o1[0]).abs().amax(-1) / o1[0].abs().amax(-1)
        err_p = (out_p - o1[0]).abs().amax(-1) / o1[0].abs().amax(-1)
        max_rel = float(torch.maximum(err, err_p).max())
        assert max_rel <= 2e-3, f"sequence-split output differs from the single-GPU decode: {max_rel:.3e}"
    algo_rank = count * PAGE * H_KV * BYTES_PER_UNIT
    peak, _ = measured_peak_gbs()
    res.update(us_per_layer_step=float(allt[:, 2].max()), per_rank_step_us=allt[:, 2].tolist(),
               us_per_layer_step_graph=float(allt[:, 3].max()),
               us_per_layer_step_nccl=float(allt[:, 0].max()), per_rank_step_us_nccl=allt[:, 0].tolist(), per_rank_kernel_us=allt[:, 1].tolist(),
               per_rank_achieved_GBps=[algo_rank / u / 1e3 for u in allt[:, 1].tolist()],
               frac_of_hbm_peak_per_rank=algo_rank / float(allt[:, 1].max()) / 1e3 / peak,
               collective="one kernel per rank: 32 x 130 float32 stored into every rank's buffer over NVLink, flag, bounded wait, merge "
                          "(us_per_layer_step; _graph: the step's three launches replayed as one CUDA graph); NCCL all_gather_into_tensor + "
                          "merge kernel (us_per_layer_step_nccl)",
               max_rel_err_vs_single_gpu=max_rel, peer_exchange_error=p2p_error)
    return res


# ------------------------------------------------------------------------------------------------
# Secondary workload (not the headline line): benchmark configuration 5, K4 spectral keys, one GPU
# ------------------------------------------------------------------------------------------------

def config_spectral(device, rank, world, dist, steps: int = 30) -> dict:
    """Benchmark configuration 5: K4 spectral keys, B = 64 sequences x 16384 committed tokens over all ranks (64 / N per rank:
    sequences are independent, no collective), per-head 128 x 128 packs at ~2.6 bits per direction, values as in the k2b
    workload; one page set is quantized for real and copied to every sequence (distinct memory).  The bound of this kernel
    is max(bytes at the HBM peak, decoder product at the sustained tensor peak)."""
    import torch

    from bmx_b200 import kernels as K
    from bmx_b200.rope import default_rope_tables

    dev = device
    B, T = max(1, 64 // world), 16384
    g = torch.Generator().manual_seed(5000)
    tiers = {8: 2, 6: 6, 5: 10, 4: 16, 3: 26, 2: 44}  # 104 directions with bits, 2.6 bits per direction on average
    enc, bits = [], []
    for h in range(H_KV):
        Q, _ = torch.linalg.qr(torch.randn(D, D, generator=g))
        enc.append(Q)
        by = [b for b in sorted(tiers, reverse=True) for _ in range(tiers[b])]
        bh = torch.zeros(D, dtype=torch.int32)
        bh[torch.randperm(D, generator=g)] = torch.tensor(by + [0] * (D - len(by)), dtype=torch.int32)
        bits.append(bh)
    enc, bits = torch.stack(enc), torch.stack(bits)
    pack = K.SpectralPackDev(enc, enc.clone(), bits, page=128, group=64, device=dev)
    npg = T // 128
    kpool, vpool = pack.new_pool(B * npg), K.vblock_pool(H_KV, B * npg, dev)
    k = (torch.randn(1, H_KV, T, D, generator=g) * 2).half().to(dev)
    v = torch.randn(1, H_KV, T, D, generator=g).half().to(dev)
    signs, cb = K.hadamard_signs(D, 0).to(dev), torch.tensor(K.GAUSSIAN_CODEBOOK[2]).to(dev)
    slots0 = torch.arange(npg, dtype=torch.int32, device=dev)
    K.spectral_append(pack, kpool, k, slots0, npg)
    K.vblock_append(vpool, v, signs, cb, slots0, npg)
    kpool.view(B, npg, H_KV, -1)[1:] = kpool.view(B, npg, H_KV, -1)[0]
    vpool.view(B, npg, H_KV, -1)[1:] = vpool.view(B, npg, H_KV, -1)[0]
    table = torch.arange(B * npg, dtype=torch.int32, device=dev).view(B, npg)
    n_pages = torch.full((B,), npg, dtype=torch.int32, device=dev)
    cos, sin = (t.half().contiguous() for t in default_rope_tables(ROPE_THETA, D, T + 512, device=dev))
    q = (torch.randn(B, H_KV * G, D, generator=g) / math.sqrt(D)).half().to(dev)
    kt = torch.randn(B, H_KV, 256, D, generator=g).half().to(dev)
    vt = torch.randn(B, H_KV, 256, D, generator=g).half().to(dev)
    tl = torch.full((B,), WINDOW, dtype=torch.int32, device=dev)
    ws, lut = K.spectral_decode_workspace(pack, G, B), K.v_lut_tensor(K.GAUSSIAN_CODEBOOK[2], dev)
    out = torch.empty(B, H_KV * G, D, dtype=torch.float16, device=dev)

    def step(ph):
        K.spectral_decode(pack, G, kpool, vpool, q, table, n_pages, npg, cos, sin, kt, vt, tl, lut, signs, 1 / math.sqrt(D), ws,
                          out=out, phases=ph)

    for _ in range(5):
        step(3)
    torch.cuda.synchronize()
    K.check_status(ws)
    if dist is not None:
        dist.barrier()
    ms = _event_us(lambda: step(3), steps, warm=0) / 1e3
    main_ms = _event_us(lambda: step(1), steps, warm=0) / 1e3
    K.check_status(ws)
    t = torch.tensor([ms, main_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, main_ms = t.tolist()
    units = B * H_KV * T
    per_unit = (pack.geom.block_bytes + 4352) / 128
    algo_bytes, flops = units * per_unit, units * 2.0 * 128 * 16 * math.ceil(sum(tiers.values()) / 16)
    peak, peak_kind = measured_peak_gbs()
    tf_peak = 1378.0
    try:
        tf_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops_sustained", tf_peak))
    except (OSError, ValueError):
        pass
    hbm_us, mma_us = algo_bytes / peak / 1e3, flops / tf_peak / 1e6
    return {"workload": f"K4 spectral packed-cache decode: 32 q / 8 kv heads, d=128, B={B} per GPU ({B * world} in all), T=16384 + "
                        "128-token window, per-head packs (104 of 128 directions carry 2..8 bits), V Hadamard + 2-bit Lloyd",
            "value_GBps_all_gpus": world * algo_bytes / (ms * 1e-3) / 1e9, "us_per_layer_step": ms * 1e3, "steps": steps,
            "bytes_per_token_head": per_unit, "gpu_launches_per_step": 2,
            "roofline": {"bound": "max(hbm, tensor)", "kernel": "spectral_decode_t5_kernel<4>", "kernel_us": main_ms * 1e3,
                         "hbm_us_at_peak": hbm_us, "tensor_us_at_peak": mma_us, "frac": max(hbm_us, mma_us) / (main_ms * 1e3),
                         "achieved": algo_bytes / (main_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "achieved_tflops": flops / (main_ms * 1e-3) / 1e12, "peak_tflops": tf_peak,
                         "peak_source": f"MEASURED_PEAKS.json hbm_gbs ({peak_kind}), bf16_tflops_sustained", "traffic": None}}


def config_prefill(device) -> dict:
    """Prefill attention of the k2b cache: one sequence of 16384 committed tokens + a 128-token window (32 q / 8 kv heads);
    (a) the last 32, 512 and 2048 positions as one query block (a follow-up turn, a chunk of a chunked prefill), (b) the
    whole prompt at once.  Timed:
    the paged kernel (pages dequantized in shared memory, no dense K / V; tcgen05, and the mma.sync kernel it succeeded)
    against the route it replaces, dequantize every page + rotate + scaled_dot_product_attention with the same causal mask.
    FLOPs counted over the visible part only."""
    import torch
    import torch.nn.functional as F

    from bmx_b200 import kernels as K
    from bmx_b200.rope import apply_rope

    T = 16384
    state, _, gen, _, _ = build_state(device, 4000, batch=1, ctx=T)
    S, H = T + WINDOW, H_KV * G
    out = {"workload": f"k2b causal prefill attention, B=1, {T} committed tokens + {WINDOW}-token window, 32 q / 8 kv heads"}
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            tf_peak = float(json.load(f).get("bf16_tflops_sustained") or 0) or None
    except (OSError, ValueError):
        tf_peak = None
    for name, n_q in (("last_32_rows", 32), ("last_512_rows", 512), ("last_2048_rows", 2048), ("whole_prompt", S)):
        q = (torch.randn(1, H, n_q, D, generator=gen, device=device) / math.sqrt(D)).half()
        o = torch.empty_like(q)
        K.k2b_prefill_select(1)  # the mma.sync kernel, for the record
        legacy_us = _event_us(lambda: state.prefill_attend(q, S - n_q, out=o), 3, warm=1)
        K.k2b_prefill_select(0)  # the tcgen05 kernel (default); few rows: the page walk shared out over CTAs + merge kernel
        paged_us = _event_us(lambda: state.prefill_attend(q, S - n_q, out=o), 3, warm=1)
        K.check_status(state.workspace)
        n_split = state.prefill_split(n_q)

        def dense():  # the product's dense route: one dequantizer kernel writes rotated fp16 K and V in place, then SDPA
            kx, vx = state.dense_kv(torch.float16)
            if n_q == S:
                return F.scaled_dot_product_attention(q, kx, vx, is_causal=True, scale=state.sm_scale, enable_gqa=True)
            mask = torch.ones(n_q, S, dtype=torch.bool, device=device).tril(S - n_q)
            return F.scaled_dot_product_attention(q, kx, vx, attn_mask=mask, scale=state.sm_scale, enable_gqa=True)

        torch.cuda.reset_peak_memory_stats(device)
        base = torch.cuda.memory_allocated(device)
        ref = dense()
        dense_peak = torch.cuda.max_memory_allocated(device) - base
        dense_us = _event_us(dense, 3, warm=0)
        err = float((o.float() - ref.float()).abs().max() / ref.float().abs().max())
        visible = n_q * (S - n_q) + n_q * (n_q + 1) // 2
        flops = 4.0 * H * D * visible
        out[name] = {"rows": n_q, "paged_kernel_us": paged_us, "paged_mma_sync_kernel_us": legacy_us, "dequantize_then_sdpa_us": dense_us,
                     "speedup": dense_us / paged_us,
                     "paged_tflops": flops / paged_us / 1e6, "peak_tflops": tf_peak,
                     "frac_of_tensor_peak": None if not tf_peak else flops / paged_us / 1e6 / tf_peak,
                     "dense_route_transient_bytes": int(dense_peak), "paged_route_transient_bytes": 0,
                     "max_rel_diff_between_routes": err, "page_walk_shares": n_split, "gpu_launches": 1 if n_split == 1 else 2}
        del q, o, ref
    return out


def config_latency_b1(device) -> dict:
    """The shape bmx's own kernel tables are quoted on: one sequence (B = 1), 32 q / 8 kv heads, context 2k / 8k / 32k / 128k,
    one attention layer-call; k2b with a rank-16 basis per head and 128-token pages (the configuration of its fastest
    published kernel), window of 128 fp16 tokens.  Microseconds per decode step (both kernels), replayed from a CUDA graph,
    CUDA events.  The published figures beside them were measured by bmx's author on another GPU (GH200) with bmx's Triton
    kernel: context, not a like-for-like ratio."""
    import torch

    from bmx_b200 import kernels as K
    from bmx_b200.engine import K2bLayerState
    from bmx_b200.rope import apply_rope, default_rope_tables

    rank, W = 16, 128
    published_gh200_ms = {2048: 0.079, 8192: 0.241, 32768: 0.935, 131072: 3.709}
    gen = torch.Generator(device=device).manual_seed(6000)
    basis = torch.zeros(H_KV * D, rank, device=device)
    for h in range(H_KV):
        Q, R = torch.linalg.qr(torch.randn(D, rank, generator=gen, device=device))
        basis[h * D:(h + 1) * D] = Q * torch.sign(torch.diagonal(R))
    out = {"workload": "k2b decode latency, B=1, 32 q / 8 kv heads, rank-16 per-head basis, 128-token pages and window",
           "published_reference_ms_on_gh200": {str(k): v for k, v in published_gh200_ms.items()}}
    peak, _ = measured_peak_gbs()
    per_unit = 64 + 4 + 32 + 2 + 2 * rank  # residual nibbles, scales, value codes, norm, fp16 coefficients
    for T in (2048, 8192, 32768, 131072):
        total = T + W
        cos, sin = default_rope_tables(ROPE_THETA, D, total + 256, device=device)
        geom = K.k2b_geom(H_KV, G, PAGE, rank, GROUP, H_KV)
        st = K2bLayerState(geom, 1, total + 256, W, device, cos.half(), sin.half())
        st.set_basis(basis)
        decay = torch.arange(1, rank + 1, device=device).float() ** -1.5
        coef = torch.randn(1, H_KV, total, rank, generator=gen, device=device) * decay
        k_pre = (torch.einsum("bhtr,hcr->bhtc", coef, basis.view(H_KV, D, rank)) + 0.1 * torch.randn(1, H_KV, total, D, generator=gen, device=device)).half()
        v = torch.randn(1, H_KV, total, D, generator=gen, device=device).half()
        st.append(k_pre, apply_rope(k_pre.float(), cos[:total], sin[:total]).half(), v)
        assert st.committed == T and st.tail_len == W
        q = (torch.randn(1, H_KV * G, D, generator=gen, device=device) / math.sqrt(D)).half()
        o = torch.empty(1, H_KV * G, D, dtype=torch.float16, device=device)
        st.decode(q, out=o)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            st.decode(q, out=o)
        us = _event_us(graph.replay, 200)
        K.check_status(st.workspace)
        algo = T * H_KV * per_unit
        out[str(T)] = {"us_per_layer_step": us, "algorithmic_bytes": algo, "GBps": algo / us / 1e3, "frac_of_hbm_peak": algo / us / 1e3 / peak}
        del st, k_pre, v, coef
    return out


def run_hf(args) -> None:
    """`--workload hf`: per-token decode latency of a random-init Llama-shaped model (Llama-3.1-8B layer dimensions, four
    layers, small vocabulary) with PackedStreamingCache (k2b) against DynamicCache: prefill 8192 tokens at B = 4, then time
    single-token forwards with CUDA events.  bmx measures the same for its own classes in scripts/profile_decode_ab.py and
    reports host overhead, not the kernel, as what dominates there.  Only time is compared: a random-init model's keys have
    none of the structure the codecs rely on.  Prints one JSON line."""
    import torch
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM

    from bmx_b200.packed_streaming import PackedStreamingCache
    from bmx_b200.recipes import spec_pair

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the bmxk kernels have no CPU path")
    layers, batch, context, steps, window = 4, 4, 8192, min(args.steps, 32), 128
    dev = torch.device("cuda:0")
    cfg = LlamaConfig(vocab_size=1024, hidden_size=4096, intermediate_size=14336, num_hidden_layers=layers, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, max_position_embeddings=context + steps + 64, rope_theta=500000.0)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(dev).half().eval()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (batch, context + steps + 3), generator=g).to(dev)

    def run(make_cache, attach, graphed=False):
        cache = make_cache()
        ctx = cache.attach(model) if attach else None
        step = (lambda x: model(x, past_key_values=cache, use_cache=True))
        if graphed:
            from bmx_b200.graphed import GraphedDecoder

            decoder = GraphedDecoder(model, cache)
            step = decoder.step
        try:
            with torch.no_grad():
                pos = 0
                p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                p0.record()
                while pos < context:  # prefill in chunks
                    n = min(2048, context - pos)
                    model(ids[:, pos:pos + n], past_key_values=cache, use_cache=True)
                    pos += n
                p1.record()
                torch.cuda.synchronize()
                prefill_ms.append(p0.elapsed_time(p1))
                for t in range(3):
                    step(ids[:, pos + t:pos + t + 1])
                pos += 3
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                e0.record()
                for t in range(steps):
                    step(ids[:, pos + t:pos + t + 1])
                e1.record()
                torch.cuda.synchronize()
                if graphed:
                    assert decoder.replays >= steps, (decoder.replays, decoder.eager_steps)
                return e0.elapsed_time(e1) / steps, (time.perf_counter() - t0) * 1e3 / steps
        finally:
            if ctx is not None:
                cache.detach()

    k_spec, v_spec = spec_pair("k2b_ph", rank=32, group=64)
    prefill_ms = []  # one entry per run below, in order: the 8192-token prompt in four 2048-token blocks (first run: with warm-up costs)
    dense = {}
    for impl in ("sdpa", "eager"):
        model.config._attn_implementation = impl
        ms, wall = run(lambda: DynamicCache(config=cfg), attach=False)
        dense[impl] = {"ms_per_token": ms, "wall_ms_per_token": wall, "prompt_ms": prefill_ms[-1]}
    model.config._attn_implementation = "sdpa"
    packed_ms, packed_wall = run(lambda: PackedStreamingCache(cfg, k_spec, v_spec, recent_window=window), attach=True)
    graph_ms, graph_wall = run(lambda: PackedStreamingCache(cfg, k_spec, v_spec, recent_window=window), attach=True, graphed=True)
    run(lambda: PackedStreamingCache(cfg, k_spec, v_spec, recent_window=window, prefill_route="dense"), attach=True)
    dense_ms = min(v["ms_per_token"] for v in dense.values())
    print(json.dumps({"metric": "hf_decode_ms_per_token", "model": f"Llama-3.1-8B layer shape x {layers} layers, random init, fp16",
                      "batch": batch, "context": context, "steps": steps, "dynamic_cache": dense,
                      "packed_streaming_cache_k2b": {"ms_per_token": packed_ms, "wall_ms_per_token": packed_wall},
                      "packed_streaming_cache_k2b_whole_step_graph": {"ms_per_token": graph_ms, "wall_ms_per_token": graph_wall},
                      "prompt_ms_packed_cache": {"paged_prefill_kernel": prefill_ms[3], "dequantize_then_sdpa": prefill_ms[4],
                                                 "note": "quantize-on-append of every page included; blocks of 2048 rows"},
                      "per_layer_us": {"dynamic": dense_ms * 1e3 / layers, "packed": packed_ms * 1e3 / layers,
                                       "packed_graph": graph_ms * 1e3 / layers}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--ctx", type=int, default=CTX, help="committed tokens per sequence (smaller cases for profiling)")
    ap.add_argument("--batch", type=int, default=16, help="sequences of --workload append (smaller cases for profiling)")
    ap.add_argument("--workload", default="k2b", choices=["k2b", "spectral", "append", "rtn", "prefill", "latency", "hf"],
                    help="k2b: the headline line (carries the other configurations under `configs`); spectral: the K4 spectral "
                         "cache alone, append / rtn: those configurations alone (one GPU, for profiling); hf: per-token latency "
                         "under a random-init Hugging Face model")
    args = ap.parse_args()
    assert args.ctx % PAGE == 0 and args.ctx >= PAGE
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "spectral":
        if rank == 0:
            import torch

            if not torch.cuda.is_available():
                raise SystemExit("bench.py: no CUDA device; the bmxk kernels have no CPU path")
            print(json.dumps(config_spectral(torch.device("cuda", 0), 0, 1, None, steps=min(args.steps, 50))), flush=True)
        return
    if args.workload in ("append", "rtn", "prefill", "latency"):
        if rank == 0:
            import torch

            if not torch.cuda.is_available():
                raise SystemExit("bench.py: no CUDA device; the bmxk kernels have no CPU path")
            dev0 = torch.device("cuda", 0)
            fn = {"append": lambda: config_append(dev0, B=args.batch), "rtn": lambda: config_rtn(dev0),
                  "prefill": lambda: config_prefill(dev0), "latency": lambda: config_latency_b1(dev0)}[args.workload]
            print(json.dumps(fn()), flush=True)
        return
    if args.workload == "hf":
        if rank == 0:
            run_hf(args)
        return
    run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
