"""Device-resident state of one attention layer's packed k2b cache, batched over sequences.

This is the B200-native counterpart of the state bmx keeps per `PackedStreamingLayer`
(bmx: src/bmx/cache/packed_streaming.py:321-446): committed tokens live as packed pages in a page
pool, the most recent `recent_window .. recent_window + page` tokens live as fp16 in a window
buffer, and the flush schedule is bmx's (`compute_flush_schedule`, src/bmx/cache/streaming.py:144).
Differences by design: pages are written by one CUDA launch straight into the layout the decode
kernel reads (no per-page Python dicts, no re-stacking), all sequences of a batch advance in lock
step, and a decode step is two launches with no allocation.
"""

from __future__ import annotations

import math

import torch

from . import kernels as K
from .schedule import compute_flush_schedule

HEAD_DIM = K.HEAD_DIM


def fit_basis(geom, k_pre_page: torch.Tensor) -> torch.Tensor:
    """Rank-r right singular vectors of the first page of pre-RoPE keys -> (h_kv*128, rank) float32, as bmx fits them
    on the first flush and then freezes them (bmx: src/bmx/decomp/lrs.py:35-41, src/bmx/cache/packed_streaming.py:513-516).
    One basis over all heads, or one per head.  k_pre_page: (h_kv, page, 128), or (batch, h_kv, page, 128): bmx keeps one
    cache per sequence; a batched state shares one basis, fitted on the first pages of all its sequences stacked (the
    same thing at batch 1)."""
    x = k_pre_page.float()
    if x.dim() == 4:
        x = x.permute(1, 0, 2, 3).reshape(x.shape[1], x.shape[0] * x.shape[2], x.shape[3])
    if geom.n_coef_heads == 1:
        M = x.permute(1, 0, 2).reshape(x.shape[1], geom.h_kv * HEAD_DIM)
        return torch.linalg.svd(M, full_matrices=False)[2][: geom.rank].mT.contiguous()
    return torch.cat([torch.linalg.svd(x[h], full_matrices=False)[2][: geom.rank].mT for h in range(geom.h_kv)], 0).contiguous()


def dequant_value_blocks(vpool: torch.Tensor, slots: torch.Tensor, codebook: torch.Tensor, signs: torch.Tensor) -> torch.Tensor:
    """Value-only page blocks -> float32 (n, 128 tokens, h_kv, 128): codebook level / sqrt(d), inverse Hadamard,
    signs, norm (bmx: src/bmx/cache/codecs.py:639-649).  Off the decode path (prefill, the dequantized-resident
    cache): the codes come from the exporter kernel, the rest is a few torch ops."""
    h_kv, dev = vpool.shape[1], vpool.device
    idx, norm = K.vblock_export(vpool, slots)
    codes = torch.stack([(idx >> (2 * k)) & 3 for k in range(4)], -1).reshape(idx.shape[0], 128, h_kv, HEAD_DIM).long()
    lev = codebook[codes] / math.sqrt(HEAD_DIM)
    H = torch.tensor([[1.0]], device=dev)
    while H.shape[0] < HEAD_DIM:
        H = torch.cat([torch.cat([H, H], 1), torch.cat([H, -H], 1)], 0)
    return (lev @ (H / math.sqrt(HEAD_DIM))) * signs * norm.float().unsqueeze(-1)


class K2bLayerState:
    """Packed pages + fp16 recent window of one layer for `batch` sequences of equal length."""

    # callable (k_src, n_pages) -> (batch, n_pages * page, rank) float32 that replaces the append kernel's own projection
    # (a basis spanning heads that other GPUs hold: dist.HeadShardedK2bLayer); None: the kernel projects
    project = None

    def __init__(self, geom, batch: int, max_tokens: int, recent_window: int, device, rope_cos: torch.Tensor,
                 rope_sin: torch.Tensor, *, codebook=None, v_seed: int = 0, pre_rope: bool = True):
        assert rope_cos.dtype == torch.float16 and rope_cos.shape[1] == HEAD_DIM and rope_cos.shape[0] >= 128
        self.geom, self.batch, self.device = geom, batch, torch.device(device)
        self.page, self.W, self.pre_rope = geom.page, recent_window, pre_rope
        self.max_pages = max(1, math.ceil(max_tokens / geom.page))
        self.pool = K.K2bPool(geom, batch * self.max_pages, self.device)
        self.page_table = torch.arange(batch * self.max_pages, dtype=torch.int32, device=self.device).view(batch, -1)
        self.n_pages_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.tail_len_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.append_cnt = torch.zeros(batch, dtype=torch.int32, device=self.device)  # scratch of window_append_devpos
        self.tail_cap = recent_window + geom.page
        shape = (batch, geom.h_kv, self.tail_cap, HEAD_DIM)
        self.k_win = torch.zeros(shape, dtype=torch.float16, device=self.device)      # post-RoPE keys
        self.v_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.k_pre_win = torch.zeros(shape, dtype=torch.float16, device=self.device)  # pre-RoPE keys (page source)
        self.rope_cos, self.rope_sin = rope_cos, rope_sin
        cb = tuple(codebook) if codebook is not None else K.GAUSSIAN_CODEBOOK[geom.vbits]
        self.codebook = torch.tensor(cb, dtype=torch.float32, device=self.device)
        self.v_lut = K.v_lut_tensor(cb, self.device)
        self.signs = K.hadamard_signs(HEAD_DIM, v_seed).to(self.device)
        self.basis_f32: torch.Tensor | None = None
        self.basis_f16: torch.Tensor | None = None
        self.workspace = K.decode_workspace(geom, batch, self.max_pages, self.device)
        self.committed = 0   # tokens held as packed pages (per sequence)
        self.tail_len = 0    # tokens held in the fp16 window (per sequence)
        self.sm_scale = 1.0 / math.sqrt(HEAD_DIM)

    # ---- frozen key basis -------------------------------------------------------------------
    def set_basis(self, basis_f32: torch.Tensor) -> None:
        """(h_kv*128, rank) float32 basis, frozen from now on (bmx: packed_streaming.py:513-520)."""
        g = self.geom
        assert basis_f32.shape == (g.h_kv * HEAD_DIM, g.rank)
        self.basis_f32 = basis_f32.to(self.device, torch.float32).contiguous()
        self.basis_f16 = self.basis_f32.half().contiguous()

    def fit_basis(self, k_pre_page: torch.Tensor) -> None:
        """Rank-r right singular vectors of the first page, as bmx fits them on the first flush
        (bmx: src/bmx/decomp/lrs.py:35-41).  k_pre_page: (h_kv, page, 128) or (batch, h_kv, page, 128)."""
        basis = fit_basis(self.geom, k_pre_page)
        self.set_basis(basis)

    def ensure_pages(self, n_more: int) -> None:
        """Grows the page pool (doubling) so that n_more further pages per sequence fit."""
        need = self.committed // self.page + n_more
        if need <= self.max_pages:
            return
        new_max = max(need, 2 * self.max_pages)
        old_pool, old_table, used = self.pool, self.page_table, self.committed // self.page
        self.pool = K.K2bPool(self.geom, self.batch * new_max, self.device)
        self.page_table = torch.arange(self.batch * new_max, dtype=torch.int32, device=self.device).view(self.batch, -1)
        if used:
            src = old_table[:, :used].reshape(-1).long()
            dst = self.page_table[:, :used].reshape(-1).long()
            self.pool.pages[dst] = old_pool.pages[src]
            self.pool.coefs[dst] = old_pool.coefs[src]
        self.max_pages = new_max

    # ---- append -----------------------------------------------------------------------------
    def _commit_pages(self, k_src: torch.Tensor, v_src: torch.Tensor, n_pages: int) -> None:
        """Quantizes the first n_pages pages of (batch, h_kv, T, 128) sources into the next slots."""
        if self.basis_f32 is None:
            self.fit_basis(k_src[:, :, : self.page])
        if v_src.dtype != k_src.dtype:
            v_src = v_src.to(k_src.dtype)
        if k_src.stride() != v_src.stride() or k_src.stride(3) != 1:
            k_src, v_src = k_src.contiguous(), v_src.contiguous()
        self.ensure_pages(n_pages)
        p0 = self.committed // self.page
        slots = self.page_table[:, p0:p0 + n_pages].contiguous().view(-1)
        if self.project is None:
            K.k2b_append(self.pool, k_src, v_src, self.basis_f32, self.signs, self.codebook, slots, n_pages)
        else:  # the projection onto a basis that spans heads held elsewhere (dist.HeadShardedK2bLayer)
            K.k2b_append_coefs(self.pool, k_src, v_src, self.project(k_src, n_pages), self.basis_f32, self.signs, self.codebook, slots,
                               n_pages)
        self.committed += n_pages * self.page
        self.n_pages_dev.fill_(self.committed // self.page)

    # ---- committing pages with device-side arguments only (steps replayed as CUDA graphs) --------------------
    @property
    def graph_commit_ok(self) -> bool:
        """True when commit_from_windows() needs nothing from the host: the basis is frozen and projected by the kernel."""
        return self.basis_f32 is not None and self.project is None

    def commit_from_windows(self, slots: torch.Tensor, n_pages: int) -> None:
        """Quantizes the first n_pages pages held in the windows into `slots` (device int32, sequence-major).  Launches
        only: counters and windows are advanced by the caller (window_shift on the device, committed / tail_len on the host)."""
        K.k2b_append(self.pool, self.k_pre_win if self.pre_rope else self.k_win, self.v_win, self.basis_f32, self.signs, self.codebook,
                     slots, n_pages)

    def append(self, k_pre: torch.Tensor | None, k_post: torch.Tensor, v: torch.Tensor) -> None:
        """Appends n new tokens per sequence: (batch, h_kv, n, 128) tensors (fp16 or bf16).

        k_pre is the pre-RoPE key (the page source when the cache quantizes pre-RoPE keys); k_post
        is the RoPE'd key that attention over the recent window uses.
        """
        src_k = k_pre if self.pre_rope else k_post
        n = k_post.shape[2]
        total = self.committed + self.tail_len + n
        new_commit = compute_flush_schedule(total, self.W, self.page)
        if n == 1 and new_commit <= self.committed:  # the common decode step: one token into the window
            K.window_append(k_post, v, src_k, self.k_win, self.v_win, self.k_pre_win, self.tail_len_dev, self.tail_len)
            self.tail_len += 1
            return
        if n == 1 and self.tail_len < self.tail_cap:
            # a streaming step that commits pages: the token goes into the window like any other, then whole pages are
            # quantized straight out of the windows (no concatenation) and the remaining tokens move to the front
            K.window_append(k_post, v, src_k, self.k_win, self.v_win, self.k_pre_win, self.tail_len_dev, self.tail_len)
            self.tail_len += 1
            n_flush = (new_commit - self.committed) // self.page
            self._commit_pages(self.k_pre_win if self.pre_rope else self.k_win, self.v_win, n_flush)
            off = n_flush * self.page
            rest = self.tail_len - off
            K.window_shift(self.k_win, self.v_win, self.k_pre_win, off, rest, self.tail_len_dev)  # one launch, sets the device-side length
            self.tail_len = rest
            return
        # general path: window ++ new tokens, commit whole pages, keep the rest as the new window
        t = self.tail_len
        if t:
            src_k = torch.cat([self.k_pre_win[:, :, :t].to(src_k.dtype), src_k], 2)
            k_post = torch.cat([self.k_win[:, :, :t].to(k_post.dtype), k_post], 2)
            v = torch.cat([self.v_win[:, :, :t].to(v.dtype), v], 2)
        n_flush = (new_commit - self.committed) // self.page
        if n_flush > 0:
            self._commit_pages(src_k, v, n_flush)
        off = n_flush * self.page
        rest = k_post.shape[2] - off
        assert rest <= self.tail_cap
        self.k_win[:, :, :rest] = k_post[:, :, off:]
        self.v_win[:, :, :rest] = v[:, :, off:]
        self.k_pre_win[:, :, :rest] = src_k[:, :, off:]
        self.tail_len = rest
        self.tail_len_dev.fill_(rest)

    # ---- decode -----------------------------------------------------------------------------
    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None, partial_out: torch.Tensor | None = None,
               phases: int = 3, pos_offset: int = 0) -> torch.Tensor:
        """q (batch, heads, 128) fp16 -> attention output (batch, heads, 128) over pages + window.  pos_offset: rotary
        position of this state's first committed token (a rank that holds a later part of a split sequence)."""
        max_pages = self.max_pages if self.committed else 0  # nothing committed yet: window only
        return K.k2b_decode(self.pool, q, self.basis_f16, self.page_table, self.n_pages_dev, max_pages,
                            self.rope_cos, self.rope_sin, self.k_win, self.v_win, self.tail_len_dev, self.v_lut,
                            self.signs, self.sm_scale, self.workspace, out=out, partial_out=partial_out, pos_offset=pos_offset,
                            phases=phases)

    def prefill_attend(self, q: torch.Tensor, q_pos0: int, out: torch.Tensor | None = None) -> torch.Tensor | None:
        """Causal attention of q (batch, heads, n_q, 128) fp16 at positions q_pos0 .. over everything held (pages + window),
        page by page, never materialising dense K / V (bmx dequantizes every page first: src/bmx/cache/chunked_attention.py
        :320-395).  Returns None when this state has no such kernel (64-token pages): the caller takes the dense route."""
        if type(self) is not K2bLayerState or self.geom.layout != 1 or self.geom.n_q_groups not in (1, 2, 4, 8):
            return None
        return K.k2b_prefill(self.pool, q, q_pos0, self.basis_f16, self.page_table, self.n_pages_dev, self.rope_cos, self.rope_sin,
                             self.k_win, self.v_win, self.tail_len_dev, self.v_lut, self.signs, self.sm_scale,
                             self.workspace.view(torch.int32), out=out, n_split=self.prefill_split(q.shape[2]))

    def prefill_split(self, n_q: int) -> int:
        """Shares of the page walk per block of query positions.  One CTA per (block, KV head, sequence) fills the GPU only
        for blocks of ~600 rows and more; below that the pages are shared out.  The kernel's time is (waves of CTAs) x (pages
        per share + the CTA's set-up, about four pages' worth): the number of shares (16 at most) that makes it smallest.  With a
        wave or more of whole walks the split is left alone (its partial records would only add traffic)."""
        pp = 128 // self.geom.n_q_groups
        ctas = -(-n_q // pp) * self.geom.h_kv * self.batch
        n_sm = torch.cuda.get_device_properties(self.device).multi_processor_count
        pages = self.committed // self.page
        if ctas >= n_sm:  # a wave or more of whole walks: the shares' records and their merge would only add traffic
            return 1
        best, best_cost = 1, None
        for s in range(1, 17):
            if s > 1 and pages < 4 * s:
                break
            cost = -(-ctas * s // n_sm) * (-(-pages // s) + 4)
            if best_cost is None or cost < best_cost:
                best, best_cost = s, cost
        return best

    def seq_len(self) -> int:
        return self.committed + self.tail_len

    def dense_kv(self, dtype: torch.dtype) -> tuple[torch.Tensor, torch.Tensor]:
        """Everything held as dense tensors (batch, h_kv, committed + window, 128) of the model's 16-bit type, for the
        dense prefill route: the committed pages dequantized, keys rotated at their positions, by one kernel that writes
        the final layout (4 bytes of transient per element), the fp16 window behind them."""
        assert type(self) is K2bLayerState and dtype in (torch.float16, torch.bfloat16), (type(self).__name__, dtype)
        S, n_pg = self.seq_len(), self.committed // self.page
        kd = torch.empty(self.batch, self.geom.h_kv, S, HEAD_DIM, dtype=dtype, device=self.device)
        vd = torch.empty_like(kd)
        if n_pg:
            K.k2b_dequant_dense(self.pool, self.page_table, n_pg, self.basis_f16, self.signs, self.codebook,
                                self.rope_cos if self.pre_rope else None, self.rope_sin if self.pre_rope else None, kd, vd)
        kd[:, :, self.committed:] = self.k_win[:, :, : self.tail_len]
        vd[:, :, self.committed:] = self.v_win[:, :, : self.tail_len]
        return kd, vd

    # ---- save / restore ---------------------------------------------------------------------
    def _pools(self) -> dict:
        return {"pages": self.pool.pages, "coefs": self.pool.coefs}

    def state_dict(self) -> dict:
        """Everything a later process needs to go on decoding: the used page slots (compacted, in page-table order),
        the fp16 windows, the frozen basis and the counters, as CPU tensors and ints."""
        used = self.committed // self.page
        src = self.page_table[:, :used].reshape(-1).long()
        t = self.tail_len
        return {"kind": type(self).__name__, "batch": self.batch, "page": self.page, "recent_window": self.W,
                "committed": self.committed, "tail_len": t, "pre_rope": self.pre_rope,
                "pools": {name: pool[src].cpu() for name, pool in self._pools().items()},
                "k_win": self.k_win[:, :, :t].cpu(), "v_win": self.v_win[:, :, :t].cpu(), "k_pre_win": self.k_pre_win[:, :, :t].cpu(),
                "basis_f32": None if self.basis_f32 is None else self.basis_f32.cpu()}

    def load_state_dict(self, sd: dict) -> None:
        """Restores a state saved by state_dict() into this (freshly built, same geometry) state."""
        assert sd["kind"] == type(self).__name__ and sd["batch"] == self.batch and sd["page"] == self.page
        assert sd["recent_window"] == self.W and sd["pre_rope"] == self.pre_rope and self.committed == 0 and self.tail_len == 0
        used = sd["committed"] // self.page
        self.ensure_pages(used)
        dst = self.page_table[:, :used].reshape(-1).long()
        for name, pool in self._pools().items():
            assert pool.shape[1:] == sd["pools"][name].shape[1:], f"pool {name}: block shape differs"
            pool[dst] = sd["pools"][name].to(self.device)
        t = sd["tail_len"]
        self.k_win[:, :, :t] = sd["k_win"].to(self.device)
        self.v_win[:, :, :t] = sd["v_win"].to(self.device)
        self.k_pre_win[:, :, :t] = sd["k_pre_win"].to(self.device)
        if sd["basis_f32"] is not None:
            self.set_basis(sd["basis_f32"])
        self.committed, self.tail_len = sd["committed"], t
        self.n_pages_dev.fill_(used)
        self.tail_len_dev.fill_(t)

    def packed_bytes(self) -> int:
        """Bytes of packed pages a decode step streams (per layer, all sequences)."""
        g = self.geom
        per_unit = K.page_block_bytes(g) / g.page + K.coef_block_bytes(g) * g.n_coef_heads / (g.page * g.h_kv)
        return int(self.batch * g.h_kv * self.committed * per_unit)


class SpectralLayerState(K2bLayerState):
    """Same state for the K4 spectral key codec (per-head packs): keys go to a spectral page pool, values to a
    pool of value-only blocks, and a decode step is the fused spectral kernel plus the merge kernel.

    bmx keeps such a layer as per-page dicts of tier containers and decodes it through its chunked path
    (bmx: src/bmx/cache/packed_streaming.py:491-511, 1024-1034); the flush schedule, the fp16 window and
    pre-RoPE quantization are the same as for k2b.
    """

    def __init__(self, pack: "K.SpectralPackDev", n_q_groups: int, batch: int, max_tokens: int, recent_window: int, device,
                 rope_cos: torch.Tensor, rope_sin: torch.Tensor, *, codebook=None, v_seed: int = 0):
        assert rope_cos.dtype == torch.float16 and rope_cos.shape[1] == HEAD_DIM and rope_cos.shape[0] >= 128
        assert pack.geom.page == 128, "the fused spectral decode reads 128-token pages"
        self.pack, self.n_q_groups, self.batch, self.device = pack, n_q_groups, batch, torch.device(device)
        self.geom = pack.geom
        self.page, self.W, self.pre_rope = 128, recent_window, True
        self.max_pages = max(1, math.ceil(max_tokens / self.page))
        h_kv = pack.geom.h_kv
        self.kpool = pack.new_pool(batch * self.max_pages)
        self.vpool = K.vblock_pool(h_kv, batch * self.max_pages, self.device)
        self.page_table = torch.arange(batch * self.max_pages, dtype=torch.int32, device=self.device).view(batch, -1)
        self.n_pages_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.tail_len_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.append_cnt = torch.zeros(batch, dtype=torch.int32, device=self.device)  # scratch of window_append_devpos
        self.tail_cap = recent_window + self.page
        shape = (batch, h_kv, self.tail_cap, HEAD_DIM)
        self.k_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.v_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.k_pre_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.rope_cos, self.rope_sin = rope_cos, rope_sin
        cb = tuple(codebook) if codebook is not None else K.GAUSSIAN_CODEBOOK[2]
        self.codebook = torch.tensor(cb, dtype=torch.float32, device=self.device)
        self.v_lut = K.v_lut_tensor(cb, self.device)
        self.signs = K.hadamard_signs(HEAD_DIM, v_seed).to(self.device)
        self.basis_f32 = self.basis_f16 = None  # the pack is fitted offline: nothing is frozen at the first flush
        self.workspace = K.spectral_decode_workspace(pack, n_q_groups, batch)
        self.committed = 0
        self.tail_len = 0
        self.sm_scale = 1.0 / math.sqrt(HEAD_DIM)

    def ensure_pages(self, n_more: int) -> None:
        need = self.committed // self.page + n_more
        if need <= self.max_pages:
            return
        new_max = max(need, 2 * self.max_pages)
        old_k, old_v, old_table, used = self.kpool, self.vpool, self.page_table, self.committed // self.page
        self.kpool = self.pack.new_pool(self.batch * new_max)
        self.vpool = K.vblock_pool(self.geom.h_kv, self.batch * new_max, self.device)
        self.page_table = torch.arange(self.batch * new_max, dtype=torch.int32, device=self.device).view(self.batch, -1)
        if used:
            src = old_table[:, :used].reshape(-1).long()
            dst = self.page_table[:, :used].reshape(-1).long()
            self.kpool[dst] = old_k[src]
            self.vpool[dst] = old_v[src]
        self.max_pages = new_max

    def _commit_pages(self, k_src: torch.Tensor, v_src: torch.Tensor, n_pages: int) -> None:
        if k_src.stride(3) != 1:
            k_src = k_src.contiguous()
        if v_src.stride(3) != 1:
            v_src = v_src.contiguous()
        self.ensure_pages(n_pages)
        p0 = self.committed // self.page
        slots = self.page_table[:, p0:p0 + n_pages].contiguous().view(-1)
        K.spectral_append(self.pack, self.kpool, k_src, slots, n_pages)
        K.vblock_append(self.vpool, v_src, self.signs, self.codebook, slots, n_pages)
        self.committed += n_pages * self.page
        self.n_pages_dev.fill_(self.committed // self.page)

    graph_commit_ok = True  # the pack is fitted offline: a commit needs nothing from the host

    def commit_from_windows(self, slots: torch.Tensor, n_pages: int) -> None:
        K.spectral_append(self.pack, self.kpool, self.k_pre_win, slots, n_pages)
        K.vblock_append(self.vpool, self.v_win, self.signs, self.codebook, slots, n_pages)

    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None, partial_out: torch.Tensor | None = None,
               phases: int = 3, pos_offset: int = 0) -> torch.Tensor:
        max_pages = self.max_pages if self.committed else 0
        return K.spectral_decode(self.pack, self.n_q_groups, self.kpool, self.vpool, q, self.page_table, self.n_pages_dev,
                                 max_pages, self.rope_cos, self.rope_sin, self.k_win, self.v_win, self.tail_len_dev, self.v_lut,
                                 self.signs, self.sm_scale, self.workspace, out=out, partial_out=partial_out,
                                 pos_offset=pos_offset, phases=phases)

    def _pools(self) -> dict:
        return {"kpool": self.kpool, "vpool": self.vpool}

    def dense_pages(self) -> tuple[torch.Tensor, torch.Tensor]:
        """All committed pages dequantized: pre-RoPE keys and values, float32 (batch, h_kv, committed, 128).
        Keys by the page dequantizer kernel; values from the exported codes (codebook level, inverse rotation,
        norm), as bmx: src/bmx/cache/codecs.py:639-649."""
        n_pg, h_kv = self.committed // self.page, self.geom.h_kv
        slots = self.page_table[:, :n_pg].contiguous().view(-1)
        kd = K.spectral_dequant_pages(self.pack, self.kpool, slots, want_codes=False, want_k=True)["k"]
        shp = (self.batch, n_pg * self.page, h_kv, HEAD_DIM)
        kd = kd.view(*shp).permute(0, 2, 1, 3)
        vd = dequant_value_blocks(self.vpool, slots, self.codebook, self.signs)
        vd = vd.view(self.batch, n_pg * self.page, h_kv, HEAD_DIM).permute(0, 2, 1, 3)
        return kd, vd

    def packed_bytes(self) -> int:
        return int(self.batch * self.geom.h_kv * (self.committed // self.page) * (self.geom.block_bytes + self.vpool.shape[2]))


class FullSpectralLayerState(SpectralLayerState):
    """K4 spectral keys with ONE encoder over all KV heads: enc, dec (C, C) float32 with C = h_kv * 128, bits (C,) --
    the shape of the packs bmx fits (bmx: SpectralPack, src/bmx/cache/spectral.py:174-220; quantize / dequantize
    :765-839).  The decoder product of such a pack mixes heads (C x C per token, h_kv times the work of per-head
    packs), so there is no fused kernel for it; this state runs bmx's own chunked formulation on the GPU instead:

      append   Y = M @ enc as one fp32 library GEMM over the flattened heads, then the per-direction quantizer and page
               layout of the per-head path (the append kernel is handed Y with an identity encoder: directions
               128 g .. 128 g + 127 are stored as pseudo-head g), values as in SpectralLayerState;
      decode   pages are dequantized a chunk at a time (Y_hat by the page dequantizer kernel, M_hat = Y_hat @ dec^T by a
               library GEMM), rotated at their positions and attended with a running softmax in float32, then the fp16
               window; the transient is bounded by the chunk (bmx: chunked_dequant_attention,
               src/bmx/cache/chunked_attention.py:398-530).
    """

    def __init__(self, enc: torch.Tensor, dec: torch.Tensor, bits: torch.Tensor, group: int, n_q_groups: int, batch: int, max_tokens: int,
                 recent_window: int, device, rope_cos: torch.Tensor, rope_sin: torch.Tensor, *, codebook=None, v_seed: int = 0,
                 chunk_pages: int = 32):
        C = enc.shape[0]
        assert enc.shape == dec.shape == (C, C) and bits.shape == (C,) and C % HEAD_DIM == 0
        h_kv = C // HEAD_DIM
        eye = torch.eye(HEAD_DIM).expand(h_kv, HEAD_DIM, HEAD_DIM).contiguous()
        store = K.SpectralPackDev(eye, eye, bits.reshape(h_kv, HEAD_DIM), page=128, group=group, device=device)
        super().__init__(store, n_q_groups, batch, max_tokens, recent_window, device, rope_cos, rope_sin, codebook=codebook, v_seed=v_seed)
        self.enc_full = enc.to(self.device, torch.float32).contiguous()
        self.dec_full = dec.to(self.device, torch.float32).contiguous()
        self.chunk_pages = chunk_pages

    def _commit_pages(self, k_src: torch.Tensor, v_src: torch.Tensor, n_pages: int) -> None:
        B, h_kv, T = self.batch, self.geom.h_kv, n_pages * self.page
        M = k_src[:, :, :T].permute(0, 2, 1, 3).reshape(B, T, h_kv * HEAD_DIM).float()
        Y = torch.matmul(M, self.enc_full)                       # (B, T, C) float32: direction d = 128 g + j
        y_heads = Y.view(B, T, h_kv, HEAD_DIM).permute(0, 2, 1, 3)  # pseudo-heads as a strided view, no copy
        if v_src.stride(3) != 1:
            v_src = v_src.contiguous()
        self.ensure_pages(n_pages)
        p0 = self.committed // self.page
        slots = self.page_table[:, p0:p0 + n_pages].contiguous().view(-1)
        K.spectral_append(self.pack, self.kpool, y_heads, slots, n_pages)
        K.vblock_append(self.vpool, v_src, self.signs, self.codebook, slots, n_pages)
        self.committed += n_pages * self.page
        self.n_pages_dev.fill_(self.committed // self.page)

    graph_commit_ok = False  # the encoder product is a library GEMM with temporaries: commits run through append()

    def _dense_chunk(self, p0: int, p1: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Pages p0 .. p1-1 of every sequence: pre-RoPE keys and values, float32 (batch, h_kv, tokens, 128)."""
        h_kv, n = self.geom.h_kv, p1 - p0
        slots = self.page_table[:, p0:p1].contiguous().view(-1)
        y_hat = K.spectral_dequant_pages(self.pack, self.kpool, slots, want_codes=False, want_k=True)["k"]  # (B n, page, C)
        kd = torch.matmul(y_hat, self.dec_full.t()).view(self.batch, n * self.page, h_kv, HEAD_DIM).permute(0, 2, 1, 3)
        vd = dequant_value_blocks(self.vpool, slots, self.codebook, self.signs)
        return kd, vd.view(self.batch, n * self.page, h_kv, HEAD_DIM).permute(0, 2, 1, 3)

    def dense_pages(self) -> tuple[torch.Tensor, torch.Tensor]:
        n_pg = self.committed // self.page
        parts = [self._dense_chunk(p, min(n_pg, p + self.chunk_pages)) for p in range(0, n_pg, self.chunk_pages)]
        return torch.cat([k for k, _ in parts], 2), torch.cat([v for _, v in parts], 2)

    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None, partial_out: torch.Tensor | None = None,
               phases: int = 3, pos_offset: int = 0) -> torch.Tensor:
        if partial_out is not None or phases != 3:
            raise NotImplementedError("a pack that mixes heads decodes through the chunked route: no partial states")
        from .rope import apply_rope

        B, h_kv, G = self.batch, self.geom.h_kv, self.n_q_groups
        qf = q.float().view(B, h_kv, G, HEAD_DIM) * self.sm_scale
        m = torch.full((B, h_kv, G, 1), float("-inf"), device=self.device)
        l = torch.zeros(B, h_kv, G, 1, device=self.device)
        acc = torch.zeros(B, h_kv, G, HEAD_DIM, device=self.device)

        def attend(k, v):  # (B, h_kv, n, 128) float32 each: one step of the running softmax
            nonlocal m, l, acc
            s = torch.matmul(qf, k.transpose(2, 3))
            m_new = torch.maximum(m, s.amax(-1, keepdim=True))
            w, f = torch.exp(s - m_new), torch.exp(m - m_new)
            l, acc, m = l * f + w.sum(-1, keepdim=True), acc * f + torch.matmul(w, v), m_new

        n_pg = self.committed // self.page
        for p0 in range(0, n_pg, self.chunk_pages):
            p1 = min(n_pg, p0 + self.chunk_pages)
            kd, vd = self._dense_chunk(p0, p1)
            t0, t1 = pos_offset + p0 * self.page, pos_offset + p1 * self.page
            attend(apply_rope(kd, self.rope_cos[t0:t1].float(), self.rope_sin[t0:t1].float()), vd)
        if self.tail_len:
            attend(self.k_win[:, :, : self.tail_len].float(), self.v_win[:, :, : self.tail_len].float())
        res = (acc / l).view(B, h_kv * G, HEAD_DIM)
        if out is None:
            return res.to(torch.float16)
        out.copy_(res)
        return out

    def packed_bytes(self) -> int:
        return int(self.batch * self.geom.h_kv * (self.committed // self.page) * (self.geom.block_bytes + self.vpool.shape[2]))


class RtnLayerState(K2bLayerState):
    """Same state for the plain RTN arms (bmx rtn_token / rtn_channel keys, rtn_token values): keys are quantized
    after RoPE, so there is no basis, no rotation at read and no separate page-source window.  A decode step is the RTN
    page-streaming kernel plus the merge kernel (bmx: src/bmx/cache/packed_streaming.py:904-944 dispatches this arm pair
    to fused_decode_attention_packed; quantize-on-append as :643-678)."""

    def __init__(self, geom: "K.RtnGeom", batch: int, max_tokens: int, recent_window: int, device):
        self.geom, self.batch, self.device = geom, batch, torch.device(device)
        self.page, self.W, self.pre_rope = geom.page, recent_window, False
        self.max_pages = max(1, math.ceil(max_tokens / geom.page))
        self.pool = K.RtnPool(geom, batch * self.max_pages, self.device)
        self.page_table = torch.arange(batch * self.max_pages, dtype=torch.int32, device=self.device).view(batch, -1)
        self.n_pages_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.tail_len_dev = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.append_cnt = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.tail_cap = recent_window + geom.page
        shape = (batch, geom.h_kv, self.tail_cap, HEAD_DIM)
        self.k_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.v_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.k_pre_win = self.k_win  # the page source IS the post-RoPE key: one window serves both
        self.rope_cos = self.rope_sin = None
        self.basis_f32 = self.basis_f16 = None
        self.workspace = K.rtn_workspace(geom, batch, self.max_pages, self.device)
        self.committed = 0
        self.tail_len = 0
        self.sm_scale = 1.0 / math.sqrt(HEAD_DIM)

    def ensure_pages(self, n_more: int) -> None:
        need = self.committed // self.page + n_more
        if need <= self.max_pages:
            return
        new_max = max(need, 2 * self.max_pages)
        old_pool, old_table, used = self.pool, self.page_table, self.committed // self.page
        self.pool = K.RtnPool(self.geom, self.batch * new_max, self.device)
        self.page_table = torch.arange(self.batch * new_max, dtype=torch.int32, device=self.device).view(self.batch, -1)
        if used:
            src = old_table[:, :used].reshape(-1).long()
            dst = self.page_table[:, :used].reshape(-1).long()
            self.pool.pages[dst] = old_pool.pages[src]
        self.max_pages = new_max
        self.workspace = K.rtn_workspace(self.geom, self.batch, self.max_pages, self.device)

    def _commit_pages(self, k_src: torch.Tensor, v_src: torch.Tensor, n_pages: int) -> None:
        if v_src.dtype != k_src.dtype:
            v_src = v_src.to(k_src.dtype)
        if k_src.stride() != v_src.stride() or k_src.stride(3) != 1:
            k_src, v_src = k_src.contiguous(), v_src.contiguous()
        self.ensure_pages(n_pages)
        p0 = self.committed // self.page
        slots = self.page_table[:, p0:p0 + n_pages].contiguous().view(-1)
        K.rtn_append(self.pool, k_src, v_src, slots, n_pages)
        self.committed += n_pages * self.page
        self.n_pages_dev.fill_(self.committed // self.page)

    graph_commit_ok = True

    def commit_from_windows(self, slots: torch.Tensor, n_pages: int) -> None:
        K.rtn_append(self.pool, self.k_win, self.v_win, slots, n_pages)

    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None, partial_out: torch.Tensor | None = None,
               phases: int = 3, pos_offset: int = 0) -> torch.Tensor:
        """q (batch, heads, 128) fp16 -> attention output over RTN pages + window (keys carry their rotation already, so
        pos_offset has no effect; the step always runs both kernels)."""
        max_pages = self.max_pages if self.committed else 0
        return K.rtn_decode(self.pool, q, self.page_table, self.n_pages_dev, max_pages, self.k_win, self.v_win, self.tail_len_dev,
                            self.sm_scale, self.workspace, out=out, partial_out=partial_out)

    def _pools(self) -> dict:
        return {"pages": self.pool.pages}

    def dense_pages(self) -> tuple[torch.Tensor, torch.Tensor]:
        """All committed pages dequantized (code x fp16 scale): post-RoPE keys and values, float32 (batch, h_kv, committed, 128)."""
        n_pg, h_kv = self.committed // self.page, self.geom.h_kv
        slots = self.page_table[:, :n_pg].contiguous().view(-1)
        ex = K.rtn_export(self.pool, slots, dequant=True)
        shp = (self.batch, n_pg * self.page, h_kv, HEAD_DIM)
        return ex["k_deq"].view(*shp).permute(0, 2, 1, 3), ex["v_deq"].view(*shp).permute(0, 2, 1, 3)

    def packed_bytes(self) -> int:
        return int(self.batch * self.geom.h_kv * (self.committed // self.page) * self.pool.pages.shape[2])


class DecodeStepGraph:
    """One decode step of a layer state, host buffers to host buffer, as a CUDA graph.

    The step is: one ingest kernel that reads the pinned staging buffer [q | k_post | v | k_pre] straight from host
    memory (queries to a device buffer, the token into the fp16 windows at the device-side position), the two decode
    kernels, the second of which stores the attention output straight into the pinned output buffer.  (States that
    quantize non-fp16 layouts, or zero_copy=False, use copy nodes instead: staging buffer to the device, append,
    decode, output to the host.)  None of these launches has a per-step argument (positions and page counts live in device
    memory), so the sequence is captured once and replayed; on the steps where the flush schedule commits pages
    (one in `page`) the step runs through `append` / `decode` instead.  bmx's counterpart is the Python of
    PackedStreamingLayer.update + attend per token (bmx: src/bmx/cache/packed_streaming.py:582-730, 832-1064).

    hin: pinned fp16, batch * (heads + 3 * h_kv) * 128 elements laid out as q (batch, heads, 128), then k_post, v
    and k_pre, each (batch, h_kv, 1, 128); states that quantize post-RoPE keys ignore k_pre.  hout: pinned fp16
    (batch, heads, 128).
    """

    def __init__(self, state: K2bLayerState, hin: torch.Tensor, hout: torch.Tensor, zero_copy: bool = True):
        g = state.geom
        h_kv = g.h_kv
        n_q_groups = getattr(state, "n_q_groups", None) or g.n_q_groups
        heads, B = h_kv * n_q_groups, state.batch
        nq, nk = B * heads * HEAD_DIM, B * h_kv * HEAD_DIM
        assert hin.is_pinned() and hout.is_pinned() and hin.dtype == hout.dtype == torch.float16
        assert hin.numel() == nq + 3 * nk and hout.numel() == nq
        self.state, self.hin, self.hout = state, hin, hout.view(B, heads, HEAD_DIM)
        self.din = torch.empty(nq + 3 * nk, dtype=torch.float16, device=state.device)
        self.q = self.din[:nq].view(B, heads, HEAD_DIM)
        self.k_post = self.din[nq:nq + nk].view(B, h_kv, 1, HEAD_DIM)
        self.v = self.din[nq + nk:nq + 2 * nk].view(B, h_kv, 1, HEAD_DIM)
        self.k_pre = self.din[nq + 2 * nk:].view(B, h_kv, 1, HEAD_DIM)
        self.out = torch.empty(B, heads, HEAD_DIM, dtype=torch.float16, device=state.device)
        # the kernels read the pinned staging buffer and write the pinned output themselves
        self.zero_copy = zero_copy
        self.h_q = hin[:nq].view(B, heads, HEAD_DIM)
        self.h_k_post = hin[nq:nq + nk].view(B, h_kv, 1, HEAD_DIM)
        self.h_v = hin[nq + nk:nq + 2 * nk].view(B, h_kv, 1, HEAD_DIM)
        self.h_k_pre = hin[nq + 2 * nk:].view(B, h_kv, 1, HEAD_DIM)
        self.graph: torch.cuda.CUDAGraph | None = None
        self._captured_for = None  # (max_pages, pool identity): a pool that grew invalidates the captured pointers
        self._check_key = True     # pools and tables only change on the steps that go through append()
        # the step that commits pages, as a graph of its own: slots are looked up on the device, so it has no
        # per-step argument either; valid for one (pages committed, tokens left in the window) pair and one set of pools
        self.flush_graph: torch.cuda.CUDAGraph | None = None
        self._flush_captured_for = None
        self._slots = torch.zeros(B * 4, dtype=torch.int32, device=state.device)
        self.flush_replays = 0

    def _launches(self) -> None:
        st = self.state
        if self.zero_copy:
            K.step_ingest(self.h_q, self.q, self.h_k_post, self.h_v, self.h_k_pre if st.pre_rope else self.h_k_post, st.k_win, st.v_win,
                          st.k_pre_win, st.tail_len_dev, st.append_cnt, st.workspace.view(torch.int32))
            st.decode(self.q, out=self.hout)
            return
        self.din.copy_(self.hin, non_blocking=True)
        K.window_append_devpos(self.k_post, self.v, self.k_pre if st.pre_rope else self.k_post, st.k_win, st.v_win, st.k_pre_win,
                               st.tail_len_dev, st.append_cnt, st.workspace.view(torch.int32))
        st.decode(self.q, out=self.out)
        self.hout.copy_(self.out, non_blocking=True)

    def _flush_launches(self, n_flush: int, off: int, rest: int) -> None:
        """Token in, n_flush pages quantized straight out of the windows into the next slots of every sequence, windows
        shifted, decode: the launches of append() + decode() on a flush step, with nothing that depends on the step."""
        st = self.state
        K.step_ingest(self.h_q, self.q, self.h_k_post, self.h_v, self.h_k_pre if st.pre_rope else self.h_k_post, st.k_win, st.v_win,
                      st.k_pre_win, st.tail_len_dev, st.append_cnt, st.workspace.view(torch.int32))
        slots = K.gather_next_slots(st.page_table, st.n_pages_dev, n_flush, self._slots)[: st.batch * n_flush]
        st.commit_from_windows(slots, n_flush)
        K.window_shift(st.k_win, st.v_win, st.k_pre_win, off, rest, st.tail_len_dev, st.n_pages_dev, n_flush)
        st.decode(self.q, out=self.hout)

    def _key(self):
        st = self.state
        pools = (st.pool.pages.data_ptr(),) if hasattr(st, "pool") else (st.kpool.data_ptr(), st.vpool.data_ptr())
        rope = 0 if getattr(st, "rope_cos", None) is None else st.rope_cos.data_ptr()
        return (st.max_pages if st.committed else 0, pools, rope)

    def invalidate(self) -> None:
        """Call after changing the state from outside (other RoPE tables, pools swapped): the next step re-captures."""
        self._check_key = True

    def step(self) -> None:
        """Runs one step on the current stream; the caller synchronizes the stream before reading hout."""
        st = self.state
        total = st.committed + st.tail_len + 1
        new_commit = compute_flush_schedule(total, st.W, st.page)
        if new_commit > st.committed:  # pages are committed on this step
            n_flush = (new_commit - st.committed) // st.page
            off, rest = n_flush * st.page, st.tail_len + 1 - n_flush * st.page
            fits = st.committed // st.page + n_flush <= st.max_pages and n_flush <= 4 and st.tail_len < st.tail_cap
            if self.zero_copy and st.graph_commit_ok and fits:
                want = (self._key(), n_flush, off, rest)
                if self.flush_graph is not None and self._flush_captured_for == want:
                    self.flush_graph.replay()
                    self.flush_replays += 1
                else:  # once for real, then captured for the flush steps to come
                    self._flush_launches(n_flush, off, rest)
                    torch.cuda.current_stream().synchronize()
                    self.flush_graph, self._flush_captured_for = torch.cuda.CUDAGraph(), want
                    with torch.cuda.graph(self.flush_graph):
                        self._flush_launches(n_flush, off, rest)
                st.committed, st.tail_len = new_commit, rest
                return
            self.din.copy_(self.hin, non_blocking=True)
            st.append(self.k_pre, self.k_post, self.v)
            st.decode(self.q, out=self.out)
            self.hout.copy_(self.out, non_blocking=True)
            self._check_key = True
            return
        if self._check_key and self.graph is not None and self._captured_for == self._key():
            self._check_key = False
        if self.graph is None or self._check_key:
            self._launches()  # one eager pass first: lazy initialisation must not happen inside the capture
            st.tail_len += 1
            torch.cuda.current_stream().synchronize()
            self.graph, self._captured_for = torch.cuda.CUDAGraph(), self._key()
            # the capture itself executes nothing; undo nothing
            with torch.cuda.graph(self.graph):
                self._launches()
            self._check_key = False
            return
        self.graph.replay()
        st.tail_len += 1
