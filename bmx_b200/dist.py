"""Multi-GPU partitions of the decode path (one process per GPU, torch.distributed).

Two partitions, as the path allows:
  * KV heads / sequences are independent: each rank keeps its own sequences (or KV heads) and no rank
    ever talks to another during a step (`shard_range`).
  * One long sequence: rank r owns a contiguous run of pages (`split_pages`), the last rank also owns
    the fp16 window; every rank produces the un-normalised state (max, sum, accumulator) of its part
    and ONE small exchange (heads x 130 floats per rank) precedes the merge, which is bmx's split
    merge formula applied across ranks (bmx: src/bmx/cache/triton_dequant_attention.py:409-461).
    The exchange is either an NCCL all-gather followed by the merge kernel (`exchange="nccl"`) or one
    kernel per rank that stores the state into every rank's buffer over NVLink, flags, waits and merges
    (`exchange="p2p"`, PeerExchange: no library collective in the step).
Every kernel LOADS only from its own GPU's memory; what crosses NVLink is stored into the peer's buffer.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

PART_STRIDE = 130  # max (log2 units), sum, 128 accumulators


def shard_range(n_items: int, world: int, rank: int) -> tuple[int, int]:
    """[start, end) of the items (sequences or KV heads) rank `rank` owns; sizes differ by at most one."""
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def split_pages(n_pages: int, world: int) -> list[tuple[int, int]]:
    """(first page, page count) per rank for a sequence of n_pages committed pages."""
    return [(s, e - s) for s, e in (shard_range(n_pages, world, r) for r in range(world))]


def gather_partials(part: torch.Tensor, group=None) -> torch.Tensor:
    """All-gathers each rank's (rows, 130) partial state into (world, rows, 130) on every rank."""
    world = dist.get_world_size(group)
    out = torch.empty(world * part.shape[0], *part.shape[1:], dtype=part.dtype, device=part.device)
    dist.all_gather_into_tensor(out, part.contiguous(), group=group)  # concatenated along dim 0 on every backend
    return out.view(world, *part.shape)


class HeadShardedK2bLayer:
    """KV heads of one layer split across the ranks of `group` while the key basis spans ALL heads (bmx's default: one
    (h_kv*128, rank) basis per layer, src/bmx/cache/packed_streaming.py:513-520).  Decode needs no collective: every rank
    holds the coefficients (they belong to the token, not to a head) and the pages of its own heads.  Append needs one:
    the projection Us = M @ V runs over all heads' channels, so every rank projects the channels it holds and the partial
    products are summed by one all-reduce of (batch, tokens, rank) float32 per flush.  The basis is fitted on the first
    page of all heads (one all-gather of that page, once) and every rank keeps the rows of its own heads.

    state(): a K2bLayerState over the local heads with n_coef_heads = 1; use its append / decode as usual."""

    def __init__(self, h_kv_total: int, n_q_groups: int, rank_k: int, group_k: int, batch: int, max_tokens: int, recent_window: int,
                 device, rope_cos: torch.Tensor, rope_sin: torch.Tensor, group=None, page: int = 128, v_seed: int = 0):
        from . import kernels as K
        from .engine import K2bLayerState

        self.group, self.world, self.rank = group, dist.get_world_size(group), dist.get_rank(group)
        self.h0, self.h1 = shard_range(h_kv_total, self.world, self.rank)
        assert self.h1 > self.h0, "more ranks than KV heads"
        self.h_kv_total = h_kv_total
        geom = K.k2b_geom(self.h1 - self.h0, n_q_groups, page, rank_k, group_k, 1)
        self._state = K2bLayerState(geom, batch, max_tokens, recent_window, device, rope_cos, rope_sin, v_seed=v_seed)
        self._state.project = self._project
        self._state.fit_basis = self._fit_basis

    def state(self):
        return self._state

    def set_basis(self, basis_all_heads: torch.Tensor) -> None:
        """(h_kv_total*128, rank) float32, the same on every rank: the rows of the local heads are kept."""
        self._state.set_basis(basis_all_heads[self.h0 * 128:self.h1 * 128].contiguous())

    def _fit_basis(self, k_pre_page: torch.Tensor) -> None:
        """First flush: gather the first page of every head (heads in rank order), fit one basis on all of them, as a
        single-GPU state does."""
        from . import kernels as K
        from .engine import fit_basis

        st = self._state
        x = k_pre_page.float().contiguous()  # (batch, local heads, page, 128)
        counts = [shard_range(self.h_kv_total, self.world, r) for r in range(self.world)]
        parts = [torch.empty(x.shape[0], b - a, x.shape[2], x.shape[3], device=x.device) for a, b in counts]
        dist.all_gather(parts, x, group=self.group)
        full_geom = K.k2b_geom(self.h_kv_total, st.geom.n_q_groups, st.geom.page, st.geom.rank, st.geom.group, 1)
        self.set_basis(fit_basis(full_geom, torch.cat(parts, 1)))

    def _project(self, k_src: torch.Tensor, n_pages: int) -> torch.Tensor:
        st = self._state
        T = n_pages * st.page
        M = k_src[:, :, :T].permute(0, 2, 1, 3).reshape(k_src.shape[0], T, -1).float()   # (batch, T, local channels)
        us = torch.matmul(M, st.basis_f32)                                                  # partial projection
        dist.all_reduce(us, op=dist.ReduceOp.SUM, group=self.group)
        return us.contiguous()


class PeerExchange:
    """This rank's exchange buffer plus the mappings of every other rank's (CUDA IPC, one node), for
    bmxk_xchg_merge.  Set-up is collective over `group` (one all-gather of the 64-byte handles); a step is not."""

    WAIT_LIMIT_CYCLES = 4_000_000_000  # ~2 s: a rank that never arrives ends the wait with a status word, not a hang

    def __init__(self, rows: int, device, group=None):
        import ctypes

        from ._lib import call, lib

        self.rows, self.group, self.device = rows, group, torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if dist.get_backend(group) != "nccl":
            raise RuntimeError("PeerExchange maps GPU memory between the ranks of one node: it needs the nccl backend (one rank per GPU)")
        lib()
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        self._own, self._peers, ptrs, failure = None, {}, [], None
        with torch.cuda.device(self.device):
            # Every rank goes through the same collectives whether or not its own CUDA calls succeeded: a failure is
            # gathered as a flag and raised on all ranks together, so that no rank is left waiting in a collective.
            try:
                call("bmxk_xchg_alloc", rows, self.world, ctypes.byref(own), handle)
                self._own = own.value
            except Exception as e:  # noqa: BLE001 - reported below, on every rank
                failure = f"rank {self.rank}: {e}"
            mine = torch.tensor(list(handle.raw) + [0 if failure is None else 1], dtype=torch.uint8, device=self.device)
            everyone = torch.empty(self.world * 65, dtype=torch.uint8, device=self.device)
            dist.all_gather_into_tensor(everyone, mine, group=group)
            handles = everyone.cpu().view(self.world, 65)
            if failure is None and int(handles[:, 64].sum()) == 0:
                try:
                    for r in range(self.world):
                        if r == self.rank:
                            ptrs.append(own.value)
                            continue
                        peer = ctypes.c_void_p()
                        call("bmxk_xchg_open", bytes(handles[r, :64].tolist()), ctypes.byref(peer))
                        self._peers[r] = peer.value
                        ptrs.append(peer.value)
                except Exception as e:  # noqa: BLE001
                    failure = f"rank {self.rank}: {e}"
            elif failure is None:
                failure = f"ranks {[r for r in range(self.world) if int(handles[r, 64])]} could not allocate their exchange buffer"
            agreed = torch.tensor([0 if failure is None else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MAX, group=group)
            if int(agreed.item()):
                self._release_local()
                raise RuntimeError(f"peer exchange set-up failed ({failure or 'on another rank'})")
        self._ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.step = 0
        dist.barrier(group=group)  # nobody pushes into a buffer that is not mapped everywhere yet

    def merge(self, part: torch.Tensor, out: torch.Tensor | None = None, device_step: bool = False) -> torch.Tensor:
        """part: this rank's (rows, 130) float32 state -> merged, normalised (rows, 128).  Every rank calls it once per
        step, in the same order; asynchronous on the current stream.  device_step: the kernel takes the step number from
        the buffer's own count instead of an argument, so that the launch can be captured in a CUDA graph (the caller
        then advances `step` once per replay)."""
        from . import kernels as K
        from ._lib import call

        assert part.is_cuda and part.dtype == torch.float32 and part.shape == (self.rows, PART_STRIDE) and part.is_contiguous()
        if out is None:
            out = torch.empty(self.rows, K.HEAD_DIM, dtype=torch.float16, device=part.device)
        if not device_step:
            self.step += 1
        call("bmxk_xchg_merge", part.data_ptr(), self.rows, self.rank, self.world, self._ptrs, 0 if device_step else self.step, self.WAIT_LIMIT_CYCLES,
             self.status.data_ptr(), out.data_ptr(), K._dtype_code(out), torch.cuda.current_stream().cuda_stream)
        return out

    def check(self) -> None:
        """Synchronises and raises if a wait of an earlier step ran out (names the rank that never arrived)."""
        st = self.status.cpu().tolist()
        if st[0] != 0:
            raise RuntimeError(f"peer exchange: block {st[1]} gave up waiting for rank {st[2] - 32} (step {self.step})")

    def _release_local(self) -> None:
        from ._lib import call

        with torch.cuda.device(self.device):
            for ptr in self._peers.values():
                call("bmxk_xchg_close", ptr)
            self._peers = {}
            if self._own is not None:
                call("bmxk_xchg_free", self._own)
            self._own = None

    def close(self) -> None:
        """Unmaps the peers and frees the own buffer; collective (barriers: nobody frees what others still write or map)."""
        from ._lib import call

        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for ptr in self._peers.values():
                call("bmxk_xchg_close", ptr)
            self._peers = {}
            dist.barrier(group=self.group)
        self._release_local()


class SequenceSplitDecoder:
    """Decode step of one long sequence whose committed pages are split across the ranks of `group`.

    `state` is this rank's layer state (k2b or spectral) holding ITS pages only (and the window on the last rank);
    `first_page` is the index of its first page in the whole sequence, which fixes the rotary positions.
    """

    def __init__(self, state, first_page: int, group=None, exchange: str = "nccl"):
        assert exchange in ("nccl", "p2p")
        self.state, self.first_page, self.group = state, first_page, group
        rows = state.batch * state.geom.h_kv * (getattr(state, "n_q_groups", None) or state.geom.n_q_groups)
        self.part = torch.empty(rows, PART_STRIDE, dtype=torch.float32, device=state.device)
        self.peers = PeerExchange(rows, state.device, group) if exchange == "p2p" else None

    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        from . import kernels as K

        st = self.state  # a K2bLayerState or a SpectralLayerState: same call
        st.decode(q, partial_out=self.part, pos_offset=self.first_page * st.page)
        if self.peers is not None:
            return self.peers.merge(self.part, out=out)
        gathered = gather_partials(self.part, self.group)
        return K.merge_partials(gathered, out=out)

    def capture(self, q: torch.Tensor, out: torch.Tensor) -> "torch.cuda.CUDAGraph":
        """The whole step (page-streaming kernel, local merge, peer exchange + merge) as one CUDA graph over the static
        tensors q and out; p2p exchange only (a library collective is not captured here).  One eager step runs first.
        Use replay(graph) per step: it keeps the host-side step count in line with the buffer's own."""
        assert self.peers is not None, "capture() needs exchange='p2p'"
        st = self.state
        self.decode(q, out=out)
        torch.cuda.current_stream().synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            st.decode(q, partial_out=self.part, pos_offset=self.first_page * st.page)
            self.peers.merge(self.part, out=out, device_step=True)
        return graph

    def replay(self, graph) -> None:
        graph.replay()
        self.peers.step += 1

    def close(self) -> None:
        if self.peers is not None:
            self.peers.close()
