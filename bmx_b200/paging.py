"""Page-slot allocator and a multi-sequence k2b layer state on top of it.

bmx keeps one cache object per sequence and measures the steady-state cost of a sequence by running several of them side
by side (bmx: scripts/batch_oom_sweep.py:112-178).  On the B200 path all sequences of a layer share ONE page pool: a
sequence owns whatever slots the allocator handed it, its row of the page table lists them in order, and the decode and
append kernels only ever see (pool, page table, page counts).  Sequences of different lengths join and leave; freed slots
are reused.  Memory per sequence comes from the allocator's own statistics, never from exhausting the device.
"""

from __future__ import annotations

import math

import torch

from . import kernels as K
from .schedule import compute_flush_schedule

HEAD_DIM = K.HEAD_DIM


class PageAllocator:
    """Free list over `n_slots` page slots (pure host code).  Slots of a sequence are returned in allocation order."""

    def __init__(self, n_slots: int):
        assert n_slots > 0
        self.n_slots = n_slots
        self._free = list(range(n_slots - 1, -1, -1))  # pop() hands out low slots first
        self._owned: dict[object, list[int]] = {}
        self.peak_in_use = 0

    def alloc(self, seq, n: int) -> list[int]:
        """n more slots for sequence `seq`; raises MemoryError (and changes nothing) if the pool cannot hold them."""
        if n > len(self._free):
            raise MemoryError(f"page pool exhausted: {n} slots wanted, {len(self._free)} of {self.n_slots} free")
        got = [self._free.pop() for _ in range(n)]
        self._owned.setdefault(seq, []).extend(got)
        self.peak_in_use = max(self.peak_in_use, self.in_use)
        return got

    def free(self, seq) -> int:
        """Returns every slot of `seq` to the free list; the count is returned."""
        slots = self._owned.pop(seq, [])
        self._free.extend(reversed(slots))
        return len(slots)

    def slots(self, seq) -> list[int]:
        return list(self._owned.get(seq, ()))

    @property
    def in_use(self) -> int:
        return self.n_slots - len(self._free)

    def grow(self, n_more: int) -> None:
        """The pool behind this allocator was enlarged by n_more slots (existing slots keep their numbers)."""
        self._free = list(range(self.n_slots + n_more - 1, self.n_slots - 1, -1)) + self._free
        self.n_slots += n_more


class PagedK2bLayer:
    """One attention layer's k2b cache for a changing set of sequences over one shared page pool.

    Each sequence has its own length, its own fp16 window row and its own run of page slots; all sequences share the frozen
    key basis of the layer (set with set_basis, or fitted on the first page that is ever committed).  `decode` runs one
    fused step over any subset of the live sequences.
    """

    def __init__(self, geom, n_slots: int, max_seqs: int, recent_window: int, device, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
                 *, v_seed: int = 0, max_pages_per_seq: int = 1024):
        self.geom, self.device, self.page, self.W = geom, torch.device(device), geom.page, recent_window
        self.pool = K.K2bPool(geom, n_slots, self.device)
        self.alloc = PageAllocator(n_slots)
        self.max_seqs, self.max_pages = max_seqs, max_pages_per_seq
        self.tail_cap = recent_window + geom.page
        shape = (max_seqs, geom.h_kv, self.tail_cap, HEAD_DIM)
        self.k_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.v_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.k_pre_win = torch.zeros(shape, dtype=torch.float16, device=self.device)
        self.rope_cos, self.rope_sin = rope_cos, rope_sin
        cb = K.GAUSSIAN_CODEBOOK[geom.vbits]
        self.codebook = torch.tensor(cb, dtype=torch.float32, device=self.device)
        self.v_lut = K.v_lut_tensor(cb, self.device)
        self.signs = K.hadamard_signs(HEAD_DIM, v_seed).to(self.device)
        self.basis_f32 = self.basis_f16 = None
        self.sm_scale = 1.0 / math.sqrt(HEAD_DIM)
        self._rows: dict[object, int] = {}          # sequence -> row of the window buffers
        self._free_rows = list(range(max_seqs - 1, -1, -1))
        self._committed: dict[object, int] = {}
        self._tail: dict[object, int] = {}
        self._ws: dict[int, torch.Tensor] = {}      # decode workspaces by batch size

    # ---- bookkeeping ------------------------------------------------------------------------
    def set_basis(self, basis_f32: torch.Tensor) -> None:
        self.basis_f32 = basis_f32.to(self.device, torch.float32).contiguous()
        self.basis_f16 = self.basis_f32.half().contiguous()

    def add_sequence(self, seq) -> None:
        assert seq not in self._rows, f"sequence {seq!r} is live already"
        if not self._free_rows:
            raise MemoryError(f"all {self.max_seqs} sequence rows are in use")
        self._rows[seq], self._committed[seq], self._tail[seq] = self._free_rows.pop(), 0, 0

    def drop_sequence(self, seq) -> int:
        """Ends a sequence: its page slots and its window row can be reused at once.  Returns the slots freed."""
        self._free_rows.append(self._rows.pop(seq))
        del self._committed[seq], self._tail[seq]
        return self.alloc.free(seq)

    def seq_len(self, seq) -> int:
        return self._committed[seq] + self._tail[seq]

    # ---- append -----------------------------------------------------------------------------
    def append(self, seq, k_pre: torch.Tensor, k_post: torch.Tensor, v: torch.Tensor) -> None:
        """n new tokens of one sequence, (h_kv, n, 128) each (fp16 or bf16): whole pages beyond the recent window are
        quantized into freshly allocated slots, the rest stays in the sequence's fp16 window (bmx's flush schedule)."""
        from .engine import fit_basis

        row, t, n = self._rows[seq], self._tail[seq], k_post.shape[1]
        src_k = torch.cat([self.k_pre_win[row, :, :t].to(k_pre.dtype), k_pre], 1) if t else k_pre
        post = torch.cat([self.k_win[row, :, :t].to(k_post.dtype), k_post], 1) if t else k_post
        val = torch.cat([self.v_win[row, :, :t].to(v.dtype), v], 1) if t else v
        total = self._committed[seq] + t + n
        n_flush = (compute_flush_schedule(total, self.W, self.page) - self._committed[seq]) // self.page
        if n_flush > 0:
            if self.basis_f32 is None:
                self.set_basis(fit_basis(self.geom, src_k[:, : self.page]))
            assert len(self.alloc.slots(seq)) + n_flush <= self.max_pages, "sequence longer than max_pages_per_seq pages"
            slots = torch.tensor(self.alloc.alloc(seq, n_flush), dtype=torch.int32, device=self.device)
            K.k2b_append(self.pool, src_k[None].contiguous(), val[None].to(src_k.dtype).contiguous(), self.basis_f32, self.signs,
                         self.codebook, slots, n_flush)
            self._committed[seq] += n_flush * self.page
        off = n_flush * self.page
        rest = post.shape[1] - off
        assert rest <= self.tail_cap
        self.k_win[row, :, :rest], self.v_win[row, :, :rest], self.k_pre_win[row, :, :rest] = post[:, off:], val[:, off:], src_k[:, off:]
        self._tail[seq] = rest

    # ---- decode -----------------------------------------------------------------------------
    def decode(self, seqs: list, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """q (len(seqs), heads, 128) fp16: one fused decode step over those sequences, each with its own pages and window."""
        n = len(seqs)
        rows = torch.tensor([self._rows[s] for s in seqs], device=self.device)
        max_pg = max(1, max(len(self.alloc.slots(s)) for s in seqs))
        table = torch.zeros(n, max_pg, dtype=torch.int32)
        for i, s in enumerate(seqs):
            sl = self.alloc.slots(s)
            table[i, : len(sl)] = torch.tensor(sl, dtype=torch.int32)
        n_pages = torch.tensor([len(self.alloc.slots(s)) for s in seqs], dtype=torch.int32, device=self.device)
        tail = torch.tensor([self._tail[s] for s in seqs], dtype=torch.int32, device=self.device)
        if n not in self._ws:
            self._ws[n] = K.decode_workspace(self.geom, n, max_pg, self.device)
        any_pages = bool(int(n_pages.max()))
        basis16 = self.basis_f16 if self.basis_f16 is not None else torch.zeros(self.geom.h_kv * HEAD_DIM, self.geom.rank, dtype=torch.float16,
                                                                                 device=self.device)
        return K.k2b_decode(self.pool, q, basis16, table.to(self.device), n_pages, max_pg if any_pages else 0, self.rope_cos, self.rope_sin,
                            self.k_win[rows].contiguous(), self.v_win[rows].contiguous(), tail, self.v_lut, self.signs, self.sm_scale,
                            self._ws[n], out=out)

    # ---- accounting -------------------------------------------------------------------------
    def bytes_per_slot(self) -> int:
        g = self.geom
        return g.h_kv * K.page_block_bytes(g) + g.n_coef_heads * K.coef_block_bytes(g)

    def memory_stats(self) -> dict:
        """Bytes held for the live sequences, from the allocator's own counts: packed pages actually owned, plus each
        sequence's three fp16 window rows.  `per_sequence_bytes` is the steady-state marginal cost of one more sequence of
        the mean live length (bmx measures the same quantity by co-residency, scripts/batch_oom_sweep.py:112-178)."""
        n = len(self._rows)
        window = 3 * self.geom.h_kv * self.tail_cap * HEAD_DIM * 2
        pages = self.alloc.in_use * self.bytes_per_slot()
        tokens = sum(self.seq_len(s) for s in self._rows)
        dense = 2 * self.geom.h_kv * HEAD_DIM * 2  # fp16 K and V per token
        return {"sequences": n, "slots_in_use": self.alloc.in_use, "slots_total": self.alloc.n_slots, "peak_slots_in_use": self.alloc.peak_in_use,
                "packed_page_bytes": pages, "window_bytes": n * window, "per_sequence_bytes": (pages + n * window) / n if n else 0.0,
                "tokens": tokens, "bytes_per_token": (pages + n * window) / tokens if tokens else 0.0, "dense_fp16_bytes_per_token": dense}
