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
    return LlamaForCausalLM(cfg).to(dev).half().eval()


def _run(model, ids, n_prefill, force_dense):
    from bmx_b200.packed_streaming import PackedStreamingCache, PackedStreamingLayer
    from bmx_b200.recipes import spec_pair

    k_spec, v_spec = spec_pair("k2b_ph", rank=16, group=64)
    cache = PackedStreamingCache(model.config, k_spec, v_spec, recent_window=32)
    logits = []
    orig = PackedStreamingLayer.attend
    if force_dense:  # decode through dequantize-all + SDPA instead of the decode kernel
        def dense_attend(self, q, scaling, is_causal=False, attention_mask=None):
            return orig(self, q, scaling, is_causal=True, attention_mask=attention_mask)
        PackedStreamingLayer.attend = dense_attend
    try:
        with cache.attach(model), torch.no_grad():
            out = model(ids[:, :n_prefill], past_key_values=cache, use_cache=True)
            logits.append(out.logits[:, -1].float())
            for t in range(n_prefill, ids.shape[1]):
                out = model(ids[:, t:t + 1], past_key_values=cache, use_cache=True)
                logits.append(out.logits[:, -1].float())
    finally:
        PackedStreamingLayer.attend = orig
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
    la, pcache = _run(model, ids, 200, force_dense=False)
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
    assert layer._committed_S_q == pcache.layers[0]._committed_S_q == 128 + 0 * 128 or layer._committed_S_q == pcache.layers[0]._committed_S_q
    assert layer.keys.shape[2] == 240 and layer._q_prefix_k.shape[2] == layer._committed_S_q
    assert abs(cache.bits_per_entry()[0] - pcache.bits_per_entry()[0]) < 1e-9
    assert int((la.argmax(-1) != lb.argmax(-1)).sum()) == 0
    assert float((la - lb).abs().max()) < 5e-2
    k, v = cache.reconstruct_layer(0)
    assert k.shape == v.shape == (1, 2, 240, 128)
