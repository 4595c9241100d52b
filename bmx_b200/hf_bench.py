"""Per-token decode latency of a Hugging Face model with PackedStreamingCache against DynamicCache.

    python -m bmx_b200.hf_bench [--layers 4] [--batch 4] [--context 8192] [--steps 32]

A random-init Llama-shaped model with Llama-3.1-8B layer dimensions (hidden 4096, 32 query / 8 KV heads,
head_dim 128, MLP 14336) and a small vocabulary; `--layers` of them (weights are not available offline, and
the per-layer cost is what is compared).  Prefill `--context` tokens, then time `--steps` single-token
forwards with CUDA events.  bmx measures the same thing for its own classes in
scripts/profile_decode_ab.py:316-439 and reports host overhead, not the kernel, as what dominates there
(docs/2026-07-05-authoritative-vm-results.md:193-216).  Prints one JSON line.  Only time is compared: a random-init
model's keys have none of the structure the codecs rely on, so its logits say nothing about accuracy (the tests
compare the decode kernel with the dense path on the same pages instead).
"""

from __future__ import annotations

import argparse
import json
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--window", type=int, default=128)
    args = ap.parse_args()

    import torch
    from transformers import DynamicCache, LlamaConfig, LlamaForCausalLM

    from .packed_streaming import PackedStreamingCache
    from .recipes import spec_pair

    if not torch.cuda.is_available():
        raise SystemExit("hf_bench: no CUDA device; the bmxk kernels have no CPU path")
    dev = torch.device("cuda:0")
    cfg = LlamaConfig(vocab_size=1024, hidden_size=4096, intermediate_size=14336, num_hidden_layers=args.layers,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                      max_position_embeddings=args.context + args.steps + 64, rope_theta=500000.0)
    torch.manual_seed(0)
    model = LlamaForCausalLM(cfg).to(dev).half().eval()
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.context + args.steps + 3), generator=g).to(dev)

    def run(make_cache, attach):
        cache = make_cache()
        ctx = cache.attach(model) if attach else None
        try:
            with torch.no_grad():
                # prefill in chunks, so that the dense transient of the packed cache's prefill path stays small
                pos = 0
                while pos < args.context:
                    n = min(2048, args.context - pos)
                    model(ids[:, pos:pos + n], past_key_values=cache, use_cache=True)
                    pos += n
                for t in range(3):  # warm-up steps
                    model(ids[:, pos + t:pos + t + 1], past_key_values=cache, use_cache=True)
                pos += 3
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                e0.record()
                for t in range(args.steps):
                    out = model(ids[:, pos + t:pos + t + 1], past_key_values=cache, use_cache=True)
                e1.record()
                torch.cuda.synchronize()
                wall = (time.perf_counter() - t0) * 1e3 / args.steps
                return e0.elapsed_time(e1) / args.steps, wall, out.logits[:, -1].float()
        finally:
            if ctx is not None:
                cache.detach()

    k_spec, v_spec = spec_pair("k2b_ph", rank=32, group=64)
    dense = {}
    for impl in ("sdpa", "eager"):  # the dense cache with both stock attention implementations
        model.config._attn_implementation = impl
        ms, wall, _ = run(lambda: DynamicCache(config=cfg), attach=False)
        dense[impl] = {"ms_per_token": ms, "wall_ms_per_token": wall}
    model.config._attn_implementation = "sdpa"
    dense_ms = min(v["ms_per_token"] for v in dense.values())
    packed_ms, packed_wall, _ = run(lambda: PackedStreamingCache(cfg, k_spec, v_spec, recent_window=args.window), attach=True)
    print(json.dumps({
        "metric": "hf_decode_ms_per_token", "model": f"Llama-3.1-8B layer shape x {args.layers} layers, random init, fp16",
        "batch": args.batch, "context": args.context, "steps": args.steps,
        "dynamic_cache": dense,
        "packed_streaming_cache_k2b": {"ms_per_token": packed_ms, "wall_ms_per_token": packed_wall},
        "per_layer_us": {"dynamic": dense_ms * 1e3 / args.layers, "packed": packed_ms * 1e3 / args.layers},
    }), flush=True)


if __name__ == "__main__":
    main()
