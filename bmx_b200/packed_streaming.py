"""Packed streaming KV cache for Hugging Face models, on the bmxk CUDA kernels.

Drop-in for bmx's `PackedStreamingCache` / `PackedStreamingLayer`
(bmx: src/bmx/cache/packed_streaming.py:310-1222): same constructor arguments, same attach / detach /
context-manager protocol, same registered attention name ("chunked_dequant") and mask function, same
flush schedule and bits-per-entry accounting.  What differs is underneath: committed tokens live in
a device page pool written by one quantize-on-append launch per flush, and a decode step is the
split-KV dequant-attention kernel reading those pages; there are no per-page Python dicts and no
CPU or PyTorch fallback for decode.  Arm pairs without a CUDA decode kernel raise.
"""

from __future__ import annotations

import weakref

import torch
import torch.nn.functional as F
from transformers.cache_utils import Cache, DynamicLayer
from transformers.masking_utils import ALL_MASK_ATTENTION_FUNCTIONS, sdpa_mask
from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

from . import kernels as K
from .engine import FullSpectralLayerState, K2bLayerState, RtnLayerState, SpectralLayerState
from .rope import apply_rope, rope_tables_from_config
from .schedule import cache_bits_per_entry, codec_bpe, compute_flush_schedule, scale_bits
from .specs import FUSED_PAIRS, CacheCodecSpec

_ATTN_NAME = "chunked_dequant"
HEAD_DIM = K.HEAD_DIM

# Process-shared growing RoPE tables keyed by (device, rope parameters): every layer of every cache on
# one model reads the same fp16 pair (bmx: src/bmx/cache/packed_streaming.py:79-113).
_ROPE_SHARED: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def resolve_text_config(model_config):
    tc = getattr(model_config, "text_config", None)
    return tc if tc is not None and hasattr(tc, "num_attention_heads") else model_config


def resolve_decoder_layers(model):
    inner = getattr(model, "model", None)
    if inner is not None:
        lm = getattr(inner, "language_model", None)
        if lm is not None and hasattr(lm, "layers"):
            return lm.layers
        if hasattr(inner, "layers"):
            return inner.layers
    raise ValueError(f"cannot locate decoder layers of {type(model).__name__}")


def resolve_k_capture_module(self_attn):
    """Module whose forward output is the pre-RoPE key: k_norm when the family normalises per head
    (Qwen3), else k_proj (bmx: src/bmx/cache/hf_compat.py:60-96)."""
    has_q, has_k = hasattr(self_attn, "q_norm"), hasattr(self_attn, "k_norm")
    assert has_q == has_k, "attention has only one of q_norm / k_norm; capture point ambiguous"
    for alt in ("q_layernorm", "k_layernorm", "qk_norm"):
        assert not hasattr(self_attn, alt), f"unsupported pre-RoPE norm '{alt}'"
    return self_attn.k_norm if has_k else self_attn.k_proj


def _rope_key(config, device) -> tuple:
    return (str(device), float(getattr(config, "rope_theta", 0.0) or 0.0), int(getattr(config, "head_dim", 0) or 0),
            int(getattr(config, "hidden_size", 0)), int(getattr(config, "num_attention_heads", 0)),
            str(getattr(config, "rope_parameters", getattr(config, "rope_scaling", None))))


def shared_rope(config, upto: int, device) -> tuple[torch.Tensor, torch.Tensor]:
    """fp16 cos/sin (>= upto, head_dim) shared by all layers; grows by doubling."""
    config = resolve_text_config(config)
    key = _rope_key(config, device)
    cur = _ROPE_SHARED.get(key)
    if cur is None or cur[0].shape[0] < upto:
        n = max(upto, 2 * (cur[0].shape[0] if cur else 0), 1024)
        cos, sin = rope_tables_from_config(config, n, device=device)
        _ROPE_SHARED[key] = (cos.half().contiguous(), sin.half().contiguous())
    return _ROPE_SHARED[key]


def chunked_attention_forward(module, query, key, value, attention_mask, scaling, dropout=0.0, **kwargs):
    """Registered attention function: (b, H, n_q, d) query -> ((b, n_q, H*d), None), computed from the
    packed state on `module._packed_layer`; the dense key/value arguments are ignored
    (bmx: src/bmx/cache/packed_streaming.py:270-298)."""
    assert hasattr(module, "_packed_layer"), "PackedStreamingCache.attach(model) must be called before forward"
    layer = module._packed_layer
    n_q = query.shape[2]
    out = layer.attend(query, scaling, is_causal=(n_q > 1), attention_mask=attention_mask)  # (b, H, n_q, d)
    b, H, n_q, d = out.shape
    return out.transpose(1, 2).reshape(b, n_q, H * d).to(query.dtype), None


ALL_ATTENTION_FUNCTIONS.register(_ATTN_NAME, chunked_attention_forward)
ALL_MASK_ATTENTION_FUNCTIONS.register(_ATTN_NAME, sdpa_mask)


class SpectralHeadPacks:
    """Per-head K4 spectral packs of one layer: enc, dec (h_kv, 128, 128) float32 with Y = M @ enc[h] and
    M_hat = Y_hat @ dec[h].T, bits (h_kv, 128) from {0, 2, 3, 4, 5, 6, 8}, group = token group of the scales
    (the fields of bmx's SpectralPack that the codec reads, src/bmx/cache/spectral.py:174-220, one per head)."""

    def __init__(self, enc: torch.Tensor, dec: torch.Tensor, bits: torch.Tensor, group: int = 64,
                 tiers: tuple = (0, 2, 3, 4, 5, 6, 8), dec_tier: int | None = None):
        assert enc.shape == dec.shape and enc.dim() == 3 and enc.shape[1:] == (HEAD_DIM, HEAD_DIM) and bits.shape == enc.shape[:2]
        self.enc, self.dec, self.bits, self.group = enc.float(), dec.float(), bits.to(torch.int32), int(group)
        # accounting only: the tier grid the bits were allocated on, and the tier threshold up to which `dec` was put
        # through the int8 round trip when the pack was materialised (None: none was; bmx: SpectralPack.dec_tier)
        self.tiers, self.dec_tier = tuple(tiers), dec_tier

    @property
    def c_used(self) -> int:
        """Decoder columns that carry bits, over all heads (bmx: SpectralPack.c_used, src/bmx/cache/spectral.py:208-211)."""
        return int((self.bits != 0).sum())

    def c_int8(self, tier_threshold: int) -> int:
        """Used decoder columns held as int8 at that threshold (bmx: src/bmx/cache/spectral.py:213-220)."""
        return int(((self.bits > 0) & (self.bits <= tier_threshold)).sum())


class SpectralFullPack:
    """A K4 spectral pack of one layer with ONE encoder over all KV heads, the shape bmx fits: enc, dec (C, C) float32,
    Y = M @ enc over the concatenated heads, M_hat = Y_hat @ dec.T, bits (C,) (bmx: SpectralPack,
    src/bmx/cache/spectral.py:174-220).  Served by the chunked route (engine.FullSpectralLayerState), not by the
    fused decode kernel."""

    def __init__(self, enc: torch.Tensor, dec: torch.Tensor, bits: torch.Tensor, group: int = 64,
                 tiers: tuple = (0, 2, 3, 4, 5, 6, 8), dec_tier: int | None = None):
        C = enc.shape[0]
        assert enc.shape == dec.shape == (C, C) and C % HEAD_DIM == 0 and bits.shape == (C,)
        self.enc, self.dec, self.bits, self.group = enc.float(), dec.float(), bits.to(torch.int32), int(group)
        self.tiers, self.dec_tier = tuple(tiers), dec_tier

    @property
    def c_used(self) -> int:
        return int((self.bits != 0).sum())

    def c_int8(self, tier_threshold: int) -> int:
        return int(((self.bits > 0) & (self.bits <= tier_threshold)).sum())


def check_rtn_specs(k_spec: CacheCodecSpec, v_spec: CacheCodecSpec) -> None:
    """What the RTN kernels cover: post-RoPE keys of 2..4 bits, 2-bit values, groups of 32 / 64 / 128."""
    if k_spec.pre_rope:
        raise NotImplementedError("RTN keys are quantized after RoPE (bmx routes pre-RoPE RTN keys to its chunked path: "
                                  "src/bmx/cache/packed_streaming.py:904-912); set pre_rope=False")
    if not 2 <= k_spec.bits <= 4 or v_spec.bits != 2:
        raise NotImplementedError(f"RTN kernels: key bits {k_spec.bits} must be 2..4 and value bits {v_spec.bits} must be 2")
    if k_spec.group not in (32, 64, 128) or v_spec.group not in (32, 64, 128):
        raise NotImplementedError(f"RTN kernels: groups {k_spec.group} / {v_spec.group} must be 32, 64 or 128")


class PackedStreamingLayer(DynamicLayer):
    """Per-layer packed cache: page pool + frozen key basis + fp16 recent window."""

    # Prompt attention over a k2b cache has two routes.  "paged": the kernel that dequantizes one page at a time in shared
    # memory (no dense K / V for the context); "dense": dequantize every committed page (one kernel writes rotated K and V
    # in the model's 16-bit type), then the library's scaled_dot_product_attention (what bmx does, in float32 and with
    # five times the transient).  The dense route pays for the dequantization of the whole context once, the paged kernel
    # once per block of 128 / G query positions, but the library's attention is slow on few rows against a long context.
    # Measured at 16384 committed tokens, B = 1: 512 new rows 0.37 ms paged against 0.67 ms dense, 2048 rows 1.30 against
    # 1.15 ms, the whole prompt 5.0 against 1.76 ms; under a model at B = 4 (context growing through the prompt) 2048-row
    # blocks are 1.6 x faster paged.  "auto" takes the paged kernel for blocks of up to PAGED_MAX_ROWS rows (a follow-up
    # turn, a chunk of a chunked prefill), and for longer blocks once the dense route's transient would pass
    # DENSE_PREFILL_BUDGET bytes.
    PREFILL_ROUTES = ("auto", "paged", "dense")
    PAGED_MAX_ROWS = 2048
    DENSE_PREFILL_BUDGET = 1 << 30
    DENSE_BYTES_PER_ELEMENT = 12  # measured peak: K and V in the model's 16-bit type (4) + the attention call's own workspace

    def __init__(self, k_spec: CacheCodecSpec, v_spec: CacheCodecSpec, model_config, recent_window: int = 32,
                 pack_v: bool = True, pack_k: bool = True, pack=None, prefill_route: str = "auto"):
        super().__init__()
        assert prefill_route in self.PREFILL_ROUTES, prefill_route
        self.prefill_route = prefill_route
        self.k_spec, self.v_spec, self.model_config = k_spec, v_spec, model_config
        if not (pack_v and pack_k):
            # bmx keeps unpacked codes in int8 / int16 containers when these are False (a debugging aid of its Triton
            # path, bmx: src/bmx/cache/packed_streaming.py:1087-1089); pages here exist in the packed form only
            raise NotImplementedError("pack_k=False / pack_v=False: this library stores codes bit-packed only")
        self.recent_window, self.pack_v, self.pack_k = recent_window, pack_v, pack_k
        kind = FUSED_PAIRS.get((k_spec.arm, v_spec.arm))
        if kind not in ("k2b", "spectral", "rtn"):
            raise NotImplementedError(
                f"no CUDA decode kernel for arms K={k_spec.arm!r} / V={v_spec.arm!r} in PackedStreamingLayer; "
                "supported: lowrank_rtn_channel + turboquant_mse_perhead (recipe 'k2b_ph'), rtn_token or rtn_channel keys "
                "with rtn_token values (recipe 'kivi'), and spectral + turboquant_mse_perhead. "
                "There is no CPU fallback.")
        if kind == "rtn":
            check_rtn_specs(k_spec, v_spec)
        if kind == "spectral" and pack is None:
            raise NotImplementedError(
                "the spectral key arm needs a pack per layer: PackedStreamingCache(..., spectral_packs={layer: pack}) with "
                "SpectralHeadPacks (one 128 x 128 encoder per head: fused decode kernel) or SpectralFullPack (one encoder over "
                "all heads: chunked route), or a pack file named by the spec's pack_path")
        self._kind, self._pack = kind, pack
        tc = resolve_text_config(model_config)
        self._h_kv = getattr(tc, "num_key_value_heads", tc.num_attention_heads)
        self._d_head = getattr(tc, "head_dim", None) or tc.hidden_size // tc.num_attention_heads
        self._n_q_groups = tc.num_attention_heads // self._h_kv
        if self._d_head != HEAD_DIM:
            raise NotImplementedError(f"head_dim={self._d_head}: the bmxk kernels are built for head_dim 128")
        self._g = pack.group if kind == "spectral" else k_spec.group  # spectral: the pack's own fitted group
        self._page = max(self._g, (128 // self._g) * self._g) if self._g > 1 else 128
        self._k_pre: torch.Tensor | None = None   # pre-RoPE keys captured by the hook since the last update
        self._committed_S_q = 0
        self._quant_bits_k = self._quant_bits_v = 0.0
        self.bpe_k = self.bpe_v = float("nan")
        self._k_blocks: list[tuple[int, int, int]] = []   # (page index, start, end) of committed pages
        self._v_blocks: list[tuple[int, int, int]] = []
        self._frozen_svd: tuple | None = None
        self._state: K2bLayerState | None = None
        self._batch = 0
        self._graph_mode = False  # set by GraphedDecoder around a captured / replayed single-token step
        self._graph_flush = None  # (pages, offset, tokens left) while GraphedDecoder captures a step that commits pages
        self._slots: torch.Tensor | None = None

    # ---- hooks ----------------------------------------------------------------------------------
    def stash_pre_rope(self, out: torch.Tensor) -> None:
        """k_proj / k_norm output (b, S, h_kv*d) or (b, S, h_kv, d) -> (b, h_kv, S, d) fp16, kept until update()."""
        b, S = out.shape[0], out.shape[1]
        block = out.reshape(b, S, self._h_kv, self._d_head).permute(0, 2, 1, 3).to(torch.float16)
        self._k_pre = block if self._k_pre is None else torch.cat([self._k_pre, block], dim=2)

    # ---- state ----------------------------------------------------------------------------------
    def _ensure_state(self, key_states: torch.Tensor) -> K2bLayerState:
        if self._state is None:
            self._batch = key_states.shape[0]
            cos, sin = shared_rope(self.model_config, 4096, key_states.device)
            if self._kind == "spectral":
                assert self.k_spec.pre_rope, "the spectral arm quantizes pre-RoPE keys"
                if isinstance(self._pack, SpectralFullPack):  # one encoder over all heads: the chunked route
                    assert self._pack.enc.shape[0] == self._h_kv * HEAD_DIM, "pack width differs from h_kv * head_dim"
                    self._state = FullSpectralLayerState(self._pack.enc, self._pack.dec, self._pack.bits, self._g, self._n_q_groups,
                                                         self._batch, 4096, self.recent_window, key_states.device, cos, sin,
                                                         v_seed=self.v_spec.seed)
                else:
                    dev_pack = K.SpectralPackDev(self._pack.enc, self._pack.dec, self._pack.bits, page=self._page, group=self._g,
                                                 device=key_states.device)
                    self._state = SpectralLayerState(dev_pack, self._n_q_groups, self._batch, 4096, self.recent_window,
                                                     key_states.device, cos, sin, v_seed=self.v_spec.seed)
            elif self._kind == "rtn":
                geom = K.rtn_geom(self._h_kv, self._n_q_groups, self._page, self.k_spec.arm, self.k_spec.group, self.v_spec.group,
                                  self.k_spec.bits, self.v_spec.bits)
                self._state = RtnLayerState(geom, self._batch, 4096, self.recent_window, key_states.device)
            else:
                geom = K.k2b_geom(self._h_kv, self._n_q_groups, self._page, self.k_spec.rank, self.k_spec.group, 1,
                                  self.k_spec.bits, self.v_spec.bits)
                self._state = K2bLayerState(geom, self._batch, 4096, self.recent_window, key_states.device, cos, sin,
                                            v_seed=self.v_spec.seed, pre_rope=self.k_spec.pre_rope)
            self.dtype, self.device, self.is_initialized = key_states.dtype, key_states.device, True
        return self._state

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, *args, **kwargs):
        """Appends (b, h_kv, n, d) keys/values, flushing whole pages on the reference's schedule; returns the
        fp16 window as (keys, values) for HF bookkeeping (attention reads the packed state instead)."""
        st = self._ensure_state(key_states)
        n = key_states.shape[2]
        if self._graph_mode:
            return self._update_graph_step(key_states, value_states)
        if self.k_spec.pre_rope:
            assert self._k_pre is not None and self._k_pre.shape[2] == n, (
                "k_spec.pre_rope=True but no pre-RoPE keys were captured; call cache.attach(model) before the forward")
            k_pre, self._k_pre = self._k_pre, None
        else:
            k_pre = None
        total = st.seq_len() + n
        if st.rope_cos is not None and total + 1 > st.rope_cos.shape[0]:  # the shared table grows by doubling: rarely
            st.rope_cos, st.rope_sin = shared_rope(self.model_config, total + 1, key_states.device)
        before = st.committed
        if self._frozen_svd is not None and self._kind == "k2b" and st.basis_f32 is None:
            st.set_basis(self._frozen_svd[1])  # a basis frozen elsewhere (restored state, another cache): never refit
        st.append(k_pre, key_states.to(torch.float16), value_states.to(torch.float16))
        if st.basis_f32 is not None and self._frozen_svd is None:
            self._frozen_svd = (None, st.basis_f32)
        self._account(before)
        self.keys = st.k_win[:, :, : st.tail_len]
        self.values = st.v_win[:, :, : st.tail_len]
        return self.keys, self.values

    def _account(self, committed_before: int) -> None:
        """Bookkeeping after tokens were appended: every newly committed page is charged the codec's bits per entry, the
        window 16 bits (bmx: src/bmx/cache/packed_streaming.py:680-730)."""
        st = self._state
        C = self._h_kv * self._d_head
        for pg0 in range(committed_before, st.committed, self._page):
            entries = self._page * C
            if self._kind == "spectral":  # mean bits + scales of the directions that carry any (bmx: spectral.py:602-615)
                bits = self._pack.bits.float()
                bpe_page = float(bits.mean()) + scale_bits(self._g) * float((bits > 0).float().mean())
            else:
                bpe_page = codec_bpe(self.k_spec.arm, bits=self.k_spec.bits, group=self.k_spec.group, rank=self.k_spec.rank,
                                     S=self._page, C=C)
            self._quant_bits_k += bpe_page * entries
            self._quant_bits_v += codec_bpe(self.v_spec.arm, bits=self.v_spec.bits, group=self.v_spec.group,
                                            rank=0, S=self._page, C=C, h_heads=self._h_kv) * entries
            self._k_blocks.append((pg0 // self._page, pg0, pg0 + self._page))
            self._v_blocks.append((pg0 // self._page, pg0, pg0 + self._page))
        self._committed_S_q = st.committed
        S = st.seq_len()
        if S > 0:
            self.bpe_k = (self._quant_bits_k + st.tail_len * C * 16.0) / (S * C)
            self.bpe_v = (self._quant_bits_v + st.tail_len * C * 16.0) / (S * C)

    def _update_graph_step(self, key_states: torch.Tensor, value_states: torch.Tensor):
        """The single-token, no-flush case of update() with nothing that depends on the step: the token goes into the
        fp16 window at the position held in device memory, so the launch can sit in a captured CUDA graph.  Host-side
        counters are advanced afterwards by advance_after_graph_step(), once per replay."""
        st = self._state
        assert key_states.shape[2] == 1
        k_post = key_states.to(torch.float16).contiguous()
        v = value_states.to(torch.float16).contiguous()
        if self.k_spec.pre_rope:
            assert self._k_pre is not None and self._k_pre.shape[2] == 1, "no pre-RoPE key captured for this step"
            k_src, self._k_pre = self._k_pre.contiguous(), None
        else:
            k_src = k_post
        K.window_append_devpos(k_post, v, k_src, st.k_win, st.v_win, st.k_pre_win, st.tail_len_dev, st.append_cnt,
                               st.workspace.view(torch.int32))
        if self._graph_flush is not None:  # this step commits pages: slots looked up on the device, pages quantized out of the windows
            n_flush, off, rest = self._graph_flush
            if self._slots is None:
                self._slots = torch.zeros(st.batch * 4, dtype=torch.int32, device=st.device)
            slots = K.gather_next_slots(st.page_table, st.n_pages_dev, n_flush, self._slots)[: st.batch * n_flush]
            st.commit_from_windows(slots, n_flush)
            K.window_shift(st.k_win, st.v_win, st.k_pre_win, off, rest, st.tail_len_dev, st.n_pages_dev, n_flush)
        return st.k_win, st.v_win  # the attention function reads the packed state, not these

    def advance_after_graph_step(self) -> None:
        """Host-side bookkeeping of one replayed step: window length, blended bits per entry, the window views."""
        st = self._state
        st.tail_len += 1
        C, S = self._h_kv * self._d_head, st.seq_len()
        self.bpe_k = (self._quant_bits_k + st.tail_len * C * 16.0) / (S * C)
        self.bpe_v = (self._quant_bits_v + st.tail_len * C * 16.0) / (S * C)
        self.keys, self.values = st.k_win[:, :, : st.tail_len], st.v_win[:, :, : st.tail_len]

    def graph_flush_plan(self):
        """(pages, offset, tokens left) of the commit the next single-token step makes, if that step can run without any
        per-step host argument (the state can commit out of its windows, room in the pool); None if the step commits nothing
        or has to run eagerly."""
        st = self._state
        if st is None or not st.graph_commit_ok:
            return None
        new_commit = compute_flush_schedule(st.seq_len() + 1, self.recent_window, self._page)
        n_flush = (new_commit - st.committed) // self._page
        if n_flush < 1 or n_flush > 4 or st.committed // self._page + n_flush > st.max_pages or st.tail_len >= st.tail_cap:
            return None
        return n_flush, n_flush * self._page, st.tail_len + 1 - n_flush * self._page

    def advance_after_graph_flush(self, plan) -> None:
        """Host-side bookkeeping of one replayed step that committed pages."""
        st = self._state
        n_flush, _, rest = plan
        before = st.committed
        st.committed, st.tail_len = before + n_flush * self._page, rest
        self._account(before)
        self.keys, self.values = st.k_win[:, :, : st.tail_len], st.v_win[:, :, : st.tail_len]

    def next_step_flushes(self) -> bool:
        """True if appending one more token commits a page (such a step runs the append kernels: not replayable)."""
        st = self._state
        return st is None or compute_flush_schedule(st.seq_len() + 1, self.recent_window, self._page) > st.committed

    def get_seq_length(self) -> int:
        return 0 if self._state is None else self._state.seq_len()

    # ---- attention ------------------------------------------------------------------------------
    def _dense_kv(self, dtype):
        """All committed pages dequantized (keys rotated at their positions) + the window: (b, h_kv, S, d)."""
        st = self._state
        n_pg = st.committed // self._page
        if self._kind == "k2b" and dtype in (torch.float16, torch.bfloat16):
            return st.dense_kv(dtype)
        parts_k, parts_v = [], []
        if n_pg:
            if self._kind in ("spectral", "rtn"):
                kd, vd = st.dense_pages()
            else:
                slots = st.page_table[:, :n_pg].contiguous().view(-1)
                kd, vd = K.k2b_dequant_pages(st.pool, slots, st.basis_f16, st.signs, st.codebook)
                shp = (st.batch, n_pg * self._page, self._h_kv, self._d_head)
                kd = kd.view(*shp).permute(0, 2, 1, 3)
                vd = vd.view(*shp).permute(0, 2, 1, 3)
            if self.k_spec.pre_rope:
                kd = apply_rope(kd.to(dtype), st.rope_cos[: st.committed].to(dtype), st.rope_sin[: st.committed].to(dtype))
            parts_k.append(kd.to(dtype))
            parts_v.append(vd.to(dtype))
        parts_k.append(st.k_win[:, :, : st.tail_len].to(dtype))
        parts_v.append(st.v_win[:, :, : st.tail_len].to(dtype))
        return torch.cat(parts_k, 2), torch.cat(parts_v, 2)

    @staticmethod
    def _mask_is_causal(attention_mask, n_q: int, S: int) -> bool:
        """True when the mask hides exactly the keys at positions after each query row (rows are the last n_q positions
        of S).  Boolean masks mark visible keys with True, additive ones hidden keys with a large negative number."""
        if attention_mask is None:
            return True
        m = attention_mask
        if m.dim() != 4 or m.shape[-2] != n_q or m.shape[-1] != S or m.shape[1] != 1:
            return False
        vis = m if m.dtype == torch.bool else (m > -1.0)
        want = torch.ones(n_q, S, dtype=torch.bool, device=m.device).tril(S - n_q)
        return bool((vis == want).all())

    def attend(self, q: torch.Tensor, scaling: float, is_causal: bool = False, attention_mask=None) -> torch.Tensor:
        """q (b, H, n_q, d) -> (b, H, n_q, d).  Decode (n_q == 1) runs the split-KV dequant-attention kernel;
        prefill dequantizes the pages once and calls SDPA with the model's mask, as the reference does
        (bmx: src/bmx/cache/chunked_attention.py:320-395)."""
        st = self._state
        assert st is not None, "attend() before update()"
        if q.dim() == 3:
            q = q.unsqueeze(0)
        b, H, n_q, d = q.shape
        if n_q == 1 and not is_causal:
            st.sm_scale = float(scaling)
            out = st.decode(q[:, :, 0, :].to(torch.float16).contiguous())
            return out.unsqueeze(2).to(q.dtype)
        # prefill: rows at the last n_q positions, causal.  With the model's plain causal mask (or none) the paged kernel
        # attends page by page; any other mask (padding) goes through the dequantize-everything route, as in bmx.
        S = st.seq_len()
        paged = self._kind == "k2b" and st.committed > 0 and n_q <= S and self.prefill_route != "dense"
        if paged and self.prefill_route == "auto":
            over_budget = b * st.committed * self._h_kv * self._d_head * self.DENSE_BYTES_PER_ELEMENT > self.DENSE_PREFILL_BUDGET
            paged = n_q <= self.PAGED_MAX_ROWS or over_budget
        if paged and self._mask_is_causal(attention_mask, n_q, S):
            st.sm_scale = float(scaling)
            out = st.prefill_attend(q.to(torch.float16).contiguous(), S - n_q)
            if out is not None:
                return out.to(q.dtype)
        Kd, Vd = self._dense_kv(q.dtype)
        gqa = self._n_q_groups > 1
        if attention_mask is None:  # no mask: a multi-row block is the whole prompt, causal; KV heads are shared, not copied
            return F.scaled_dot_product_attention(q, Kd, Vd, is_causal=n_q > 1, scale=scaling, enable_gqa=gqa)
        if self._mask_is_causal(attention_mask, n_q, S):  # the model's plain causal mask: no per-sequence mask, no copies of K / V
            if n_q == S:
                return F.scaled_dot_product_attention(q, Kd, Vd, is_causal=n_q > 1, scale=scaling, enable_gqa=gqa)
            mask = torch.ones(n_q, S, dtype=torch.bool, device=q.device).tril(S - n_q)
            return F.scaled_dot_product_attention(q, Kd, Vd, attn_mask=mask, scale=scaling, enable_gqa=gqa)
        Kx = Kd.repeat_interleave(self._n_q_groups, dim=1)
        Vx = Vd.repeat_interleave(self._n_q_groups, dim=1)
        return F.scaled_dot_product_attention(q, Kx, Vx, attn_mask=attention_mask, scale=scaling)


class PackedStreamingCache(Cache):
    """Cache container replicating PackedStreamingLayer across the model; drop-in `past_key_values`.

        cache = PackedStreamingCache(model.config, k_spec=k_spec, v_spec=v_spec, recent_window=128)
        with cache.attach(model):
            out = model.generate(..., past_key_values=cache)
    """

    def __init__(self, model_config, k_spec: CacheCodecSpec, v_spec: CacheCodecSpec, recent_window: int = 32,
                 pack_v: bool = True, pack_k: bool = True, spectral_packs: dict | None = None, prefill_route: str = "auto"):
        self._packs = dict(spectral_packs or {})
        self.prefill_route = prefill_route
        if k_spec.arm == "spectral" and not self._packs and k_spec.pack_path:
            # the pack file is read once here and handed out by layer index (bmx: packed_streaming.py:1086-1094)
            from .packs import load_head_packs

            tc = resolve_text_config(model_config)
            self._packs = load_head_packs(k_spec.pack_path, k_spec.budget, getattr(tc, "num_key_value_heads", tc.num_attention_heads),
                                          k_spec.dec_quant)
        wself = weakref.proxy(self)  # a strong capture would make a cycle that keeps the page pools alive

        def _make_layer():
            return PackedStreamingLayer(k_spec, v_spec, model_config, recent_window, pack_v=pack_v, pack_k=pack_k,
                                        pack=wself._pack_for_layer(len(wself.layers)), prefill_route=wself.prefill_route)

        self._make_layer = _make_layer
        super().__init__(layer_class_to_replicate=_make_layer)
        self.model_config, self.k_spec, self.v_spec = model_config, k_spec, v_spec
        self.recent_window, self.pack_v, self.pack_k = recent_window, pack_v, pack_k
        self._handles: list = []
        self._saved_impl: str | None = None
        self._model = None

    def _pack_for_layer(self, i: int):
        """Layer i's spectral packs (bmx: src/bmx/cache/packed_streaming.py:1144-1148); None for other arms."""
        if self.k_spec.arm != "spectral":
            return None
        if i not in self._packs:
            raise NotImplementedError(
                f"no spectral pack for layer {i}: pass spectral_packs={{layer: SpectralHeadPacks or SpectralFullPack}} or a "
                "pack file that holds this layer")
        return self._packs[i]

    def bits_per_entry(self):
        """(bpe_k, bpe_v): blended bits per entry averaged across layers (bmx: streaming.py:154-260)."""
        return cache_bits_per_entry(self.layers, self.k_spec)

    def memory_report(self, seq_len: int) -> dict:
        """Dense fp16 bytes vs packed (bpe-derived) bytes of the whole cache (bmx: streaming.py:263-305)."""
        bpe_k, bpe_v = self.bits_per_entry()
        cfg = resolve_text_config(self.model_config)
        h_kv = getattr(cfg, "num_key_value_heads", cfg.num_attention_heads)
        d = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        entries = cfg.num_hidden_layers * h_kv * seq_len * d
        fp16_bytes = 2 * entries * 2
        bpe_k = 16.0 if bpe_k != bpe_k else bpe_k
        bpe_v = 16.0 if bpe_v != bpe_v else bpe_v
        packed_bytes = entries * (bpe_k + bpe_v) / 8.0
        return {"fp16_bytes": float(fp16_bytes), "packed_bytes": float(packed_bytes),
                "compression": fp16_bytes / max(packed_bytes, 1e-9)}

    def attach(self, model) -> "PackedStreamingCache":
        self.detach()
        self._model = model
        self._saved_impl = model.config._attn_implementation
        model.config._attn_implementation = _ATTN_NAME
        n_layers = len(resolve_decoder_layers(model))
        while len(self.layers) < n_layers:
            self.layers.append(self._make_layer())
        for i, mlayer in enumerate(resolve_decoder_layers(model)):
            mlayer.self_attn._packed_layer = self.layers[i]
            if self.k_spec.pre_rope:
                wself = weakref.proxy(self)  # a hook that held the cache would keep its page pools alive with the model

                def k_hook(module, inp, out, i=i, wself=wself):
                    wself.layers[i].stash_pre_rope(out)

                self._handles.append(resolve_k_capture_module(mlayer.self_attn).register_forward_hook(k_hook))
        return self

    def detach(self) -> "PackedStreamingCache":
        for h in self._handles:
            h.remove()
        self._handles = []
        if self._model is not None:
            for mlayer in resolve_decoder_layers(self._model):
                if hasattr(mlayer.self_attn, "_packed_layer"):
                    del mlayer.self_attn._packed_layer
            if self._saved_impl is not None:
                self._model.config._attn_implementation = self._saved_impl
        self._model, self._saved_impl = None, None
        return self

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.detach()
        return False
