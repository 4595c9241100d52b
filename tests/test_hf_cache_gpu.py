"""PackedStreamingCache under a Hugging Face model: prefill + teacher-forced decode of a random-init
Llama-shaped model, the decode kernel against the dequantize-everything + SDPA path on the same pages
(bmx: scripts/profile_decode_ab.py:316-439 is the method: count argmax flips over 64 steps)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny_llama(dev):
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=256, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=4096,
                      rope_theta=500000.0)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to(dev).eval()  # float32: the fp16 logits of a random-init model tie exactly at some steps


def _run(model, ids, n_prefill, force_dense, prefill_route="auto"):
    from bmx_b200.packed_streaming import PackedStreamingCache, PackedStreamingLayer
    from bmx_b200.recipes import spec_pair

    k_spec, v_spec = spec_pair("k2b_ph", rank=16, group=64)
    cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32, prefill_route=prefill_route)
    logits = []
    orig = PackedStreamingLayer.attend
    from bmx_b200.engine import K2bLayerState

    orig_paged = K2bLayerState.prefill_attend
    if force_dense:  # every attention call through dequantize-all + SDPA: neither the decode nor the paged prefill kernel
        def dense_attend(self, q, scaling, is_causal=False, attention_mask=None):
            return orig(self, q, scaling, is_causal=True, attention_mask=attention_mask)
        PackedStreamingLayer.attend = dense_attend
        K2bLayerState.prefill_attend = lambda self, q, q_pos0, out=None: None
    try:
        with cache.attach(model), torch.no_grad():
            out = model(ids[:, :n_prefill], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
            for t in range(n_prefill, ids.shape[1]):
                out = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
    finally:
        PackedStreamingLayer.attend = orig
        K2bLayerState.prefill_attend = orig_paged
    return torch.stack(logits, 1), cache


def test_decode_kernel_vs_dense_path_under_hf_model():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    dev = torch.device("cuda:0")
    model = _tiny_llama(dev)
    saved_impl = model.config._attn_implementation
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 256, (1, 300 + 64), generator=g).to(dev)
    la, cache = _run(model, ids, 300, force_dense=False)
    lb, _ = _run(model, ids, 300, force_dense=True)
    assert model.config._attn_implementation == saved_impl, "detach() must restore the attention implementation"
    assert not hasattr(model.model.layers[0].self_attn, "_packed_layer")
    layer = cache.layers[0]
    # schedule: 364 tokens, window 32, page 128 -> 256 committed, 108 in the window
    assert layer._committed_S_q == 256 and layer.get_seq_length() == 364 and len(layer._k_blocks) == 2
    assert layer.keys.shape[2] == 108
    bpe_k, bpe_v = cache.bits_per_entry()
    assert 3.0 < bpe_k < 16.0 and 2.0 < bpe_v < 16.0
    flips = int((la.argmax(-1) != lb.argmax(-1)).sum())
    diff = float((la - lb).abs().max())
    assert flips == 0, f"{flips} argmax flips over {la.shape[1]} steps (max logit diff {diff:.3e})"
    assert diff < 5e-2
    rep = cache.memory_report(364)
    assert rep["compression"] > 1.0


def test_unsupported_arms_raise():
    from transformers import LlamaConfig

    from bmx_b200.packed_streaming import PackedStreamingLayer
    from bmx_b200.recipes import spec_pair

    cfg = LlamaConfig(hidden_size=512, num_attention_heads=4, num_key_value_heads=2, head_dim=128)
    k, v = spec_pair("turboquant_mse")
    with pytest.raises(NotImplementedError):
        PackedStreamingLayer(k, v, cfg)


def test_streaming_twin_matches_packed_cache_tokens():
    """Packed and dequantized-resident caches quantize the same tokens with the same kernels on the same
    schedule, so greedy decoding through either gives the same tokens and close logits
    (bmx: tests/test_packed_streaming.py:23-97)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.recipes import spec_pair
    from bmx_b200.streaming import StreamingQuantizedCache

    dev = torch.device("cuda:0")
    model = _tiny_llama(dev)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 256, (1, 200 + 40), generator=g).to(dev)
    # the twin attends its prompt over dequantized tensors with SDPA; the packed cache is put on the same route for the
    # prompt (its paged kernel agrees with it to 1e-3, which a near-tie of this random-init model's logits does not survive)
    la, pcache = _run(model, ids, 200, force_dense=False, prefill_route="dense")
    k_spec, v_spec = spec_pair("k2b_ph", rank=16, group=64)
    cache = StreamingQuantizedCache(model.config, k_spec, v_spec, recent_window=32)
    logits = []
    with cache.attach(model), torch.no_grad():
        out = model(ids[:, :200], past_key_values=cache, use_cache=True)
        logits.append(out.logits[:, -1].float())
        for t in range(200, ids.shape[1]):
            out = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
    lb = torch.stack(logits, 1)
    layer = cache.layers[0]
    assert layer._committed_S_q == pcache.layers[0]._committed_S_q == 128  # 240 tokens, window 32, page 128
    assert layer.keys.shape[2] == 240 and layer._q_prefix_k.shape[2] == layer._committed_S_q
    assert abs(cache.bits_per_entry()[0] - pcache.bits_per_entry()[0]) < 1e-9
    assert int((la.argmax(-1) != lb.argmax(-1)).sum()) == 0
    assert float((la - lb).abs().max()) < 5e-2
    k, v = cache.reconstruct_layer(0)
    assert k.shape == v.shape == (1, 2, 240, 128)


def _spectral_packs(model, seed=3):
    """Seeded per-head packs for every layer: orthogonal encoders (decoder = encoder), bits by direction index."""
    from bmx_b200.packed_streaming import SpectralHeadPacks

    cfg = model.config
    g = torch.Generator().manual_seed(seed)
    packs = {}
    tiers = [8] * 6 + [6] * 10 + [5] * 12 + [4] * 20 + [3] * 28 + [2] * 36 + [0] * 16
    for i in range(cfg.num_hidden_layers):
        enc, bits = [], []
        for h in range(cfg.num_key_value_heads):
            Q, _ = torch.linalg.qr(torch.randn(128, 128, generator=g))
            enc.append(Q)
            bits.append(torch.tensor(tiers, dtype=torch.int32)[torch.randperm(128, generator=g)])
        enc = torch.stack(enc)
        packs[i] = SpectralHeadPacks(enc, enc.clone(), torch.stack(bits), group=64)
    return packs


def test_spectral_cache_decode_kernel_vs_dense_path_under_hf_model():
    """The fused spectral decode kernel against dequantize-all + SDPA on the same pages, 64 teacher-forced steps."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.packed_streaming import PackedStreamingCache, PackedStreamingLayer
    from bmx_b200.specs import CacheCodecSpec

    dev = torch.device("cuda:0")
    model = _reference_model(dev)  # float32: fp16 logits of a random-init model tie exactly at some steps
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 256, (2, 300 + 64), generator=g).to(dev)
    k_spec = CacheCodecSpec(arm="spectral", pre_rope=True, group=64)
    v_spec = CacheCodecSpec(arm="turboquant_mse_perhead", bits=2)
    packs = _spectral_packs(model)

    def run(force_dense):
        cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32, spectral_packs=packs)
        logits = []
        orig = PackedStreamingLayer.attend
        if force_dense:
            def dense_attend(self, q, scaling, is_causal=False, attention_mask=None):
                return orig(self, q, scaling, is_causal=True, attention_mask=attention_mask)
            PackedStreamingLayer.attend = dense_attend
        try:
            with cache.attach(model), torch.no_grad():
                out = model(ids[:, :300], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
                for t in range(300, ids.shape[1]):
                    out = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
                    logits.append(out.logits[:, -1].float())
        finally:
            PackedStreamingLayer.attend = orig
        return torch.stack(logits, 1), cache

    la, cache = run(False)
    lb, _ = run(True)
    layer = cache.layers[0]
    assert layer._committed_S_q == 256 and layer.get_seq_length() == 364 and layer.keys.shape[2] == 108
    bpe_k, bpe_v = cache.bits_per_entry()  # keys: payload + the per-sequence charge of the packs' decoders (16 * 224 / 364 here)
    assert 3.0 < layer.bpe_k < 16.0 and bpe_k > layer.bpe_k + 9.0 and 2.0 < bpe_v < 16.0
    diff = float((la - lb).abs().max())
    assert diff < 5e-3
    flips = int((la.argmax(-1) != lb.argmax(-1)).sum())
    top2 = lb.topk(2, dim=-1).values
    assert flips == 0, (f"{flips} argmax flips over {la.shape[0] * la.shape[1]} steps (max logit diff {diff:.3e}, smallest top-2 gap "
                        f"{float((top2[..., 0] - top2[..., 1]).min()):.3e})")
    with pytest.raises(NotImplementedError):
        PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32)._pack_for_layer(0)


def test_spectral_streaming_twin_matches_packed_cache(tmp_path):
    """The dequantized-resident cache quantizes the same tokens with the same kernels on the same schedule as the
    packed cache, so teacher-forced logits through either agree (spectral keys, per-head packs)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.packed_streaming import PackedStreamingCache
    from bmx_b200.specs import CacheCodecSpec
    from bmx_b200.streaming import StreamingQuantizedCache

    dev = torch.device("cuda:0")
    model = _tiny_llama(dev)
    g = torch.Generator().manual_seed(6)
    ids = torch.randint(0, 256, (1, 200 + 40), generator=g).to(dev)
    k_spec = CacheCodecSpec(arm="spectral", pre_rope=True, group=64)
    v_spec = CacheCodecSpec(arm="turboquant_mse_perhead", bits=2)
    packs = _spectral_packs(model)

    def run(cache):
        logits = []
        with cache.attach(model), torch.no_grad():
            out = model(ids[:, :200], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
            for t in range(200, ids.shape[1]):
                out = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
        return torch.stack(logits, 1)

    pc = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32, spectral_packs=packs)
    sc = StreamingQuantizedCache(model.config, k_spec, v_spec, recent_window=32, spectral_packs=packs)
    la, lb = run(pc), run(sc)
    assert sc.layers[0]._committed_S_q == pc.layers[0]._committed_S_q == 128
    assert sc.layers[0].keys.shape[2] == 240
    assert abs(sc.bits_per_entry()[0] - pc.bits_per_entry()[0]) < 1e-9
    assert float((la - lb).abs().max()) < 1e-2
    no_packs = StreamingQuantizedCache(model.config, k_spec, v_spec, recent_window=32)
    with pytest.raises(NotImplementedError):
        no_packs._make_layer()
    # the same packs through a pack file named by the spec (bmx's route: pack_path + budget on the spectral spec)
    from bmx_b200.packs import save_head_packs

    path = tmp_path / "packs.safetensors"
    save_head_packs(path, packs, 2.5)
    k_file = CacheCodecSpec(arm="spectral", pre_rope=True, group=64, pack_path=str(path), budget=2.5)
    lc = run(PackedStreamingCache(model.config, k_file, v_spec, recent_window=32))
    assert torch.equal(lc, la)


# ---- against the reference's own cache: logits made by bmx's PackedStreamingCache on CPU (tests/golden/model.npz) ----

def _reference_model(dev):
    """The model of tests/golden/make_golden.py::model_level: same config, same seed, float32."""
    from transformers import LlamaForCausalLM

    from tests.golden.make_golden import tiny_llama_config

    torch.manual_seed(0)
    return LlamaForCausalLM(tiny_llama_config()).eval().to(dev)


def _teacher_forced(model, cache, ids, n_prefill=300):
    logits = []
    with cache.attach(model), torch.no_grad():
        out = model(ids[:, :n_prefill], past_key_values=cache, use_cache=True)
        logits.append(out.logits[:, -1].float())
        for t in range(n_prefill, ids.shape[1]):
            out = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
    return torch.stack(logits, 1)[0].cpu()


def _write_reference_pack_file(fx, path):
    """The spectral packs of the fixture, in bmx's own file layout: one (C, C) encoder per layer."""
    import json

    from safetensors.torch import save_file

    tensors = {}
    for i in range(2):
        enc = torch.from_numpy(fx[f"spectral_enc_l{i}"])
        tensors[f"layer{i}.enc"], tensors[f"layer{i}.dec"] = enc.contiguous(), enc.clone()
        tensors[f"layer{i}.lam"] = torch.ones(enc.shape[0])
        tensors[f"layer{i}.bits_b2.5"] = torch.from_numpy(fx[f"spectral_bits_l{i}"]).long()
    save_file(tensors, str(path))
    with open(str(path) + ".json", "w") as f:
        json.dump({"tiers": [0, 2, 3, 4, 5, 6, 8], "group": 64, "budgets": [2.5]}, f)


@pytest.mark.parametrize("recipe", ["k2b_ph", "k2b_ph_own_basis", "kivi", "rtn_c4t2", "spectral", "spectral_dec8", "spectral_full",
                                    "spectral_full_dec8"])
def test_argmax_and_accounting_match_the_reference_cache(recipe, tmp_path):
    """64 teacher-forced decode steps after a 300-token prompt: every step's argmax equals the one bmx's own
    PackedStreamingCache produced (0 flips, nothing masked), logits agree closely, and the cache-level bits per
    entry and memory report equal the reference's numbers.  `k2b_ph` replays with the key basis the reference froze;
    `k2b_ph_own_basis` fits its own (another SVD library: singular vectors may differ in sign or rotate inside a
    near-degenerate pair, the projected subspace is the same).  `spectral_full*` use packs with one dense encoder over
    both KV heads (the shape bmx fits), which go through the chunked route instead of the fused decode kernel."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.packed_streaming import PackedStreamingCache
    from bmx_b200.recipes import spec_pair
    from bmx_b200.specs import CacheCodecSpec
    from bmx_b200.streaming import StreamingQuantizedCache
    from tests.helpers import golden

    dev, fx = torch.device("cuda:0"), golden("model_full" if recipe.startswith("spectral_full") else "model")
    name = "k2b_ph" if recipe.startswith("k2b_ph") else recipe
    model = _reference_model(dev)
    if name == "k2b_ph":
        k_spec, v_spec = spec_pair("k2b_ph", rank=16, group=64)
    elif name == "kivi":
        k_spec, v_spec = spec_pair("kivi", group=64)
    elif name == "rtn_c4t2":
        k_spec, v_spec = CacheCodecSpec(arm="rtn_channel", bits=4, group=32), CacheCodecSpec(arm="rtn_token", bits=2, group=32)
    else:
        path = tmp_path / "packs.safetensors"
        _write_reference_pack_file(fx, path)
        k_spec = CacheCodecSpec(arm="spectral", pre_rope=True, group=64, pack_path=str(path), budget=2.5,
                                dec_quant="int8" if name.endswith("dec8") else "fp32")
        v_spec = CacheCodecSpec(arm="turboquant_mse_perhead", bits=2)
    ids = torch.from_numpy(fx[f"{name}_ids"]).long().to(dev)
    ref = torch.from_numpy(fx[f"{name}_logits"])
    cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32)
    if recipe == "k2b_ph":
        cache.attach(model)  # sizes the layers, so that the reference's frozen bases can be set before the first flush
        for i, layer in enumerate(cache.layers):
            layer._frozen_svd = (None, torch.from_numpy(fx[f"k2b_ph_basis_l{i}"]).to(dev))
    lg = _teacher_forced(model, cache, ids)
    assert cache.layers[0]._committed_S_q == int(fx[f"{name}_committed"])
    flips = int((lg.argmax(-1) != ref.argmax(-1)).sum())
    diff = float((lg - ref).abs().max())
    print(f"{recipe}: {flips} flips over {lg.shape[0]} steps, max |logit - reference| {diff:.3e}, reference min top-2 gap "
          f"{float(fx[name + '_min_top2_gap']):.3e}")
    assert flips == 0, f"{flips} argmax flips against the reference over {lg.shape[0]} steps (max logit diff {diff:.3e})"
    # measured: 5e-4 (RTN arms: every codec stage is elementwise), 2e-3 (spectral), 4e-3 .. 5e-3 (k2b: the projection is a
    # float32 reduction whose order differs from BLAS, so a few fp16 coefficients and residual codes move at ties)
    assert diff < (2e-3 if name in ("kivi", "rtn_c4t2") else 1e-2)
    # accounting: identical arithmetic, so equal to the last bit of a float64 sum
    bpe = cache.bits_per_entry()
    assert abs(bpe[0] - fx[f"{name}_bpe"][0]) < 1e-9 and abs(bpe[1] - fx[f"{name}_bpe"][1]) < 1e-9, (bpe, fx[f"{name}_bpe"])
    rep = cache.memory_report(ids.shape[1])
    want = fx[f"{name}_memory_report"]
    assert abs(rep["fp16_bytes"] - want[0]) < 1e-6 and abs(rep["packed_bytes"] - want[1]) < 1e-3 and abs(rep["compression"] - want[2]) < 1e-9
    if recipe.startswith("spectral_full"):
        from bmx_b200.engine import FullSpectralLayerState

        assert all(type(l._state) is FullSpectralLayerState for l in cache.layers)
    if recipe in ("kivi", "spectral_dec8", "spectral_full"):  # the dequantized-resident twin: same accounting, same tokens
        twin = StreamingQuantizedCache(model.config, k_spec, v_spec, recent_window=32)
        lt = _teacher_forced(model, twin, ids)
        tb = twin.bits_per_entry()
        assert abs(tb[0] - fx[f"{name}_twin_bpe"][0]) < 1e-9 and abs(tb[1] - fx[f"{name}_twin_bpe"][1]) < 1e-9
        assert int((lt.argmax(-1) != ref.argmax(-1)).sum()) == 0


@pytest.mark.parametrize("recipe", ["k2b_ph", "kivi"])
def test_whole_step_cuda_graph_equals_eager_decode(recipe):
    """GraphedDecoder replays a whole single-token forward (all layers) as one CUDA graph; the steps that commit a page are
    a second graph (k2b and RTN arms alike).  Teacher-forced over 300 steps (two commits inside),
    logits equal the plain eager loop's bit for bit: the same kernels run on the same data, only the launch mechanism
    differs."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bmx_b200.graphed import GraphedDecoder
    from bmx_b200.packed_streaming import PackedStreamingCache
    from bmx_b200.recipes import spec_pair

    dev = torch.device("cuda:0")
    model = _reference_model(dev)
    ids = torch.randint(0, 256, (2, 200 + 300), generator=torch.Generator().manual_seed(21)).to(dev)
    k_spec, v_spec = spec_pair(recipe, rank=16, group=64)

    def run(graphed):
        cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32)
        logits = []
        with cache.attach(model), torch.no_grad():
            model(ids[:, :200], past_key_values=cache, use_cache=True)
            dec = GraphedDecoder(model, cache)
            for t in range(200, ids.shape[1]):
                if graphed:
                    logits.append(dec.step(ids[:, t:t + 1]).float().clone())
                else:
                    logits.append(model(ids[:, t:t + 1], past_key_values=cache, use_cache=True).logits[:, -1].float())
        return torch.stack(logits, 1), cache, dec

    lg, cache_g, dec = run(True)
    le, cache_e, _ = run(False)
    # one eager step (lazy initialisation), both commits through the second graph
    assert dec.replays >= 290 and dec.flush_replays == 2 and dec.eager_steps == 1 and dec.captures <= 3, (
        dec.replays, dec.flush_replays, dec.eager_steps, dec.captures)
    assert cache_g.layers[0]._committed_S_q == cache_e.layers[0]._committed_S_q == 384
    assert cache_g.layers[0].get_seq_length() == cache_e.layers[0].get_seq_length() == 500
    assert abs(cache_g.bits_per_entry()[0] - cache_e.bits_per_entry()[0]) < 1e-12
    assert torch.equal(lg, le), f"max diff {float((lg - le).abs().max()):.3e}"
