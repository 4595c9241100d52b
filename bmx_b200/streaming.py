"""Dequantized-resident streaming cache: the twin of the packed cache that keeps the quantized-then-
dequantized prefix as dense tensors and hands `[frozen prefix | fp16 window]` to the model's ordinary
attention.  Same classes, arguments and schedule as bmx's `StreamingQuantizedLayer/Cache`
(bmx: src/bmx/cache/streaming.py:308-815); each token is quantized exactly once from its pristine
source, by the same CUDA append kernel the packed cache uses, and dequantized by the page dequantizer
(keys are rotated in float32 at their true positions, then cast, as bmx does at :495-497).
"""

from __future__ import annotations

import weakref

import torch
from transformers.cache_utils import Cache, DynamicLayer

from . import kernels as K
from .engine import dequant_value_blocks, fit_basis
from .packed_streaming import check_rtn_specs, resolve_decoder_layers, resolve_k_capture_module, resolve_text_config
from .rope import apply_rope, rope_tables_from_config
from .schedule import cache_bits_per_entry, codec_bpe, compute_flush_schedule
from .specs import FUSED_PAIRS, CacheCodecSpec

HEAD_DIM = K.HEAD_DIM


class StreamingQuantizedLayer(DynamicLayer):
    """Per-layer streaming-quantized cache; `update()` returns dense (dequantized prefix + window) K/V."""

    def __init__(self, k_spec: CacheCodecSpec, v_spec: CacheCodecSpec, model_config, recent_window: int = 32, pack=None):
        super().__init__()
        self.k_spec, self.v_spec, self.model_config, self.recent_window = k_spec, v_spec, model_config, recent_window
        self._passthrough = k_spec.arm == "fp16" and v_spec.arm == "fp16"
        self._kind = None if self._passthrough else FUSED_PAIRS.get((k_spec.arm, v_spec.arm))
        if not self._passthrough and self._kind not in ("k2b", "spectral", "rtn"):
            raise NotImplementedError(f"no CUDA codec for arms K={k_spec.arm!r} / V={v_spec.arm!r}; there is no CPU fallback")
        if self._kind == "rtn":
            check_rtn_specs(k_spec, v_spec)
        if self._kind == "spectral" and pack is None:
            raise NotImplementedError("the spectral key arm needs a pack per layer: StreamingQuantizedCache(..., "
                                      "spectral_packs={layer: SpectralHeadPacks or SpectralFullPack}) or the spec's pack_path")
        self._pack, self._pack_dev = pack, None
        tc = resolve_text_config(model_config)
        self._h_kv = getattr(tc, "num_key_value_heads", tc.num_attention_heads)
        self._d_head = getattr(tc, "head_dim", None) or tc.hidden_size // tc.num_attention_heads
        if not self._passthrough and self._d_head != HEAD_DIM:
            raise NotImplementedError(f"head_dim={self._d_head}: the bmxk kernels are built for head_dim 128")
        self._g = 1 if self._passthrough else (pack.group if self._kind == "spectral" else k_spec.group)
        self._page = max(self._g, (128 // self._g) * self._g) if self._g > 1 else 128
        self._k_pre: torch.Tensor | None = None
        self._k_pre_offset = 0
        self._q_prefix_k: torch.Tensor | None = None
        self._q_prefix_v: torch.Tensor | None = None
        self._committed_S_q = 0
        self._frozen_svd: tuple | None = None
        self._quant_bits_k = self._quant_bits_v = 0.0
        self.bpe_k = self.bpe_v = float("nan")
        self._geom = None

    def stash_pre_rope(self, out: torch.Tensor) -> None:
        b, S = out.shape[0], out.shape[1]
        block = out.reshape(b, S, self._h_kv, self._d_head).permute(0, 2, 1, 3).to(torch.float16)
        self._k_pre = block if self._k_pre is None else torch.cat([self._k_pre, block], dim=2)

    def _flush(self, k_src: torch.Tensor, v_src: torch.Tensor, start: int, end: int, dtype):
        """Quantize-then-dequantize tokens [start, end) (whole pages): returns (k_post, v) in `dtype`."""
        dev, b = k_src.device, k_src.shape[0]
        n_pg = (end - start) // self._page
        if self._kind == "spectral":
            return self._flush_spectral(k_src, v_src, start, end, dtype)
        if self._kind == "rtn":
            return self._flush_rtn(k_src, v_src, start, end, dtype)
        if self._geom is None:
            n_q_groups = resolve_text_config(self.model_config).num_attention_heads // self._h_kv
            self._geom = K.k2b_geom(self._h_kv, min(n_q_groups, 8), self._page, self.k_spec.rank, self.k_spec.group, 1,
                                    self.k_spec.bits, self.v_spec.bits)
            self._signs = K.hadamard_signs(HEAD_DIM, self.v_spec.seed).to(dev)
            self._codebook = torch.tensor(K.GAUSSIAN_CODEBOOK[self.v_spec.bits], device=dev)
        if self._frozen_svd is None:
            self._frozen_svd = (None, fit_basis(self._geom, k_src[:, :, : self._page]))
        basis = self._frozen_svd[1]
        pool = K.K2bPool(self._geom, b * n_pg, dev)
        slots = torch.arange(b * n_pg, dtype=torch.int32, device=dev)
        k_src, v_src = k_src.to(torch.float16).contiguous(), v_src.to(torch.float16).contiguous()
        K.k2b_append(pool, k_src, v_src, basis, self._signs, self._codebook, slots, n_pg)
        kd, vd = K.k2b_dequant_pages(pool, slots, basis.half().contiguous(), self._signs, self._codebook)
        shp = (b, n_pg * self._page, self._h_kv, self._d_head)
        kd, vd = kd.view(*shp).permute(0, 2, 1, 3), vd.view(*shp).permute(0, 2, 1, 3)
        if self.k_spec.pre_rope:
            cos, sin = rope_tables_from_config(self.model_config, end - start, start=start, device=dev)
            kd = apply_rope(kd, cos, sin)  # float32 tables, float32 keys, then cast
        return kd.to(dtype), vd.to(dtype)

    def _flush_rtn(self, k_src: torch.Tensor, v_src: torch.Tensor, start: int, end: int, dtype):
        """The same for the plain RTN arms: post-RoPE keys, code x fp16 scale on the way back (bmx: codecs.py:720-725, 807-811)."""
        dev, b = k_src.device, k_src.shape[0]
        n_pg = (end - start) // self._page
        if self._geom is None:
            n_q_groups = resolve_text_config(self.model_config).num_attention_heads // self._h_kv
            self._geom = K.rtn_geom(self._h_kv, min(n_q_groups, 8), self._page, self.k_spec.arm, self.k_spec.group, self.v_spec.group,
                                    self.k_spec.bits, self.v_spec.bits)
        pool = K.RtnPool(self._geom, b * n_pg, dev)
        slots = torch.arange(b * n_pg, dtype=torch.int32, device=dev)
        K.rtn_append(pool, k_src.to(torch.float16).contiguous(), v_src.to(torch.float16).contiguous(), slots, n_pg)
        ex = K.rtn_export(pool, slots, dequant=True)
        shp = (b, n_pg * self._page, self._h_kv, self._d_head)
        return ex["k_deq"].view(*shp).permute(0, 2, 1, 3).to(dtype), ex["v_deq"].view(*shp).permute(0, 2, 1, 3).to(dtype)

    def _flush_spectral(self, k_src: torch.Tensor, v_src: torch.Tensor, start: int, end: int, dtype):
        """The same for the spectral key codec: spectral append + page dequantizer for keys, value blocks for values."""
        dev, b = k_src.device, k_src.shape[0]
        n_pg = (end - start) // self._page
        full = self._pack.enc.dim() == 2  # one encoder over all heads (SpectralFullPack): library GEMMs around the same kernels
        if self._pack_dev is None:
            if full:
                eye = torch.eye(HEAD_DIM).expand(self._h_kv, HEAD_DIM, HEAD_DIM).contiguous()
                self._pack_dev = K.SpectralPackDev(eye, eye, self._pack.bits.reshape(self._h_kv, HEAD_DIM), page=self._page, group=self._g,
                                                   device=dev)
                self._enc_full, self._dec_full = self._pack.enc.to(dev), self._pack.dec.to(dev)
            else:
                self._pack_dev = K.SpectralPackDev(self._pack.enc, self._pack.dec, self._pack.bits, page=self._page, group=self._g, device=dev)
            self._signs = K.hadamard_signs(HEAD_DIM, self.v_spec.seed).to(dev)
            self._codebook = torch.tensor(K.GAUSSIAN_CODEBOOK[self.v_spec.bits], device=dev)
        slots = torch.arange(b * n_pg, dtype=torch.int32, device=dev)
        kpool, vpool = self._pack_dev.new_pool(b * n_pg), K.vblock_pool(self._h_kv, b * n_pg, dev)
        k16 = k_src.to(torch.float16)
        if full:  # Y = M @ enc over the concatenated heads; directions 128 g .. 128 g + 127 are stored as pseudo-head g
            T, C = n_pg * self._page, self._h_kv * HEAD_DIM
            Y = torch.matmul(k16[:, :, :T].permute(0, 2, 1, 3).reshape(b, T, C).float(), self._enc_full)
            K.spectral_append(self._pack_dev, kpool, Y.view(b, T, self._h_kv, HEAD_DIM).permute(0, 2, 1, 3), slots, n_pg)
        else:
            K.spectral_append(self._pack_dev, kpool, k16.contiguous(), slots, n_pg)
        K.vblock_append(vpool, v_src.to(torch.float16).contiguous(), self._signs, self._codebook, slots, n_pg)
        kd = K.spectral_dequant_pages(self._pack_dev, kpool, slots, want_codes=False, want_k=True)["k"]
        if full:
            kd = torch.matmul(kd, self._dec_full.t())
        shp = (b, n_pg * self._page, self._h_kv, self._d_head)
        kd = kd.view(*shp).permute(0, 2, 1, 3)
        vd = dequant_value_blocks(vpool, slots, self._codebook, self._signs).view(*shp).permute(0, 2, 1, 3)
        cos, sin = rope_tables_from_config(self.model_config, end - start, start=start, device=dev)
        return apply_rope(kd, cos, sin).to(dtype), vd.to(dtype)

    def _page_bpe_k(self, C: int) -> float:
        if self._kind == "spectral":  # mean bits + scales of the directions that carry any (bmx: spectral.py:602-615)
            bits = self._pack.bits.float()
            return float(bits.mean()) + 16.0 / self._g * float((bits > 0).float().mean())
        return codec_bpe(self.k_spec.arm, bits=self.k_spec.bits, group=self.k_spec.group, rank=self.k_spec.rank, S=self._page, C=C)

    def update(self, key_states, value_states, *args, **kwargs):
        keys, values = super().update(key_states, value_states, *args, **kwargs)
        if self._passthrough:
            self.bpe_k = self.bpe_v = 16.0
            return keys, values
        S, W, C = keys.shape[2], self.recent_window, self._h_kv * self._d_head
        new_S_q = compute_flush_schedule(S, W, self._page)
        if new_S_q > self._committed_S_q:
            start, end = self._committed_S_q, new_S_q
            if self.k_spec.pre_rope:
                assert self._k_pre is not None, "k_spec.pre_rope=True but no pre-RoPE keys captured; call cache.attach(model)"
                k_src = self._k_pre[:, :, start - self._k_pre_offset:end - self._k_pre_offset]
            else:
                k_src = keys[:, :, start:end]
            kq, vq = self._flush(k_src, values[:, :, start:end], start, end, keys.dtype)
            self._q_prefix_k = kq if self._q_prefix_k is None else torch.cat([self._q_prefix_k, kq], 2)
            self._q_prefix_v = vq if self._q_prefix_v is None else torch.cat([self._q_prefix_v, vq], 2)
            keys = torch.cat([self._q_prefix_k, keys[:, :, end:]], 2)
            values = torch.cat([self._q_prefix_v, values[:, :, end:]], 2)
            for _ in range(start, end, self._page):
                entries = self._page * C
                self._quant_bits_k += self._page_bpe_k(C) * entries
                self._quant_bits_v += codec_bpe(self.v_spec.arm, bits=self.v_spec.bits, group=self.v_spec.group, rank=0,
                                                S=self._page, C=C, h_heads=self._h_kv) * entries
            self._committed_S_q = end
            if self._k_pre is not None:  # write-once: committed sources are never needed again
                self._k_pre = self._k_pre[:, :, end - self._k_pre_offset:].contiguous()
                self._k_pre_offset = end
        self.keys, self.values = keys, values
        tail = S - self._committed_S_q
        self.bpe_k = (self._quant_bits_k + tail * C * 16.0) / (S * C)
        self.bpe_v = (self._quant_bits_v + tail * C * 16.0) / (S * C)
        return keys, values


class StreamingQuantizedCache(Cache):
    """Cache container replicating StreamingQuantizedLayer across the model (bmx: streaming.py:663-815)."""

    def __init__(self, model_config, k_spec: CacheCodecSpec, v_spec: CacheCodecSpec, recent_window: int = 32,
                 spectral_packs: dict | None = None):
        self._packs = dict(spectral_packs or {})
        if k_spec.arm == "spectral" and not self._packs and k_spec.pack_path:
            from .packs import load_head_packs

            tc = resolve_text_config(model_config)
            self._packs = load_head_packs(k_spec.pack_path, k_spec.budget, getattr(tc, "num_key_value_heads", tc.num_attention_heads),
                                          k_spec.dec_quant)
        wself = weakref.proxy(self)

        def _make_layer():
            pack = None
            if k_spec.arm == "spectral":  # layers are appended in order: the new layer's index is the current length
                i = len(wself.layers)
                if i not in wself._packs:
                    raise NotImplementedError(f"no spectral pack for layer {i}: pass spectral_packs={{layer: SpectralHeadPacks}}")
                pack = wself._packs[i]
            return StreamingQuantizedLayer(k_spec, v_spec, model_config, recent_window, pack=pack)

        self._make_layer = _make_layer
        super().__init__(layer_class_to_replicate=_make_layer)
        self.model_config, self.k_spec, self.v_spec, self.recent_window = model_config, k_spec, v_spec, recent_window
        self._handles: list = []

    def attach(self, model) -> "StreamingQuantizedCache":
        self.detach()
        if not self.k_spec.pre_rope:
            return self
        layers = resolve_decoder_layers(model)
        while len(self.layers) < len(layers):
            self.layers.append(self._make_layer())
        wself = weakref.proxy(self)
        for i, mlayer in enumerate(layers):
            def k_hook(module, inp, out, i=i):
                wself.layers[i].stash_pre_rope(out)

            self._handles.append(resolve_k_capture_module(mlayer.self_attn).register_forward_hook(k_hook))
        return self

    def detach(self) -> "StreamingQuantizedCache":
        for h in self._handles:
            h.remove()
        self._handles = []
        return self

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.detach()
        return False

    def reconstruct_layer(self, layer_idx: int):
        layer = self.layers[layer_idx]
        return layer.keys, layer.values

    def bits_per_entry(self):
        return cache_bits_per_entry(self.layers, self.k_spec)

    def memory_report(self, seq_len: int, h_kv: int | None = None, d_head: int | None = None) -> dict:
        bpe_k, bpe_v = self.bits_per_entry()
        cfg = resolve_text_config(self.model_config)
        h_kv = h_kv or getattr(cfg, "num_key_value_heads", cfg.num_attention_heads)
        d = d_head or (getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads)
        entries = cfg.num_hidden_layers * h_kv * seq_len * d
        fp16_bytes = 2 * entries * 2
        bpe_k = 16.0 if bpe_k != bpe_k else bpe_k
        bpe_v = 16.0 if bpe_v != bpe_v else bpe_v
        packed = entries * (bpe_k + bpe_v) / 8.0
        return {"fp16_bytes": float(fp16_bytes), "packed_bytes": float(packed), "compression": fp16_bytes / max(packed, 1e-9)}
