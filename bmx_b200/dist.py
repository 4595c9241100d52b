"""Multi-GPU partitions of the decode path (one process per GPU, torch.distributed).

Two partitions, as the path allows:
  * KV heads / sequences are independent: each rank keeps its own sequences (or KV heads) and no rank
    ever talks to another during a step (`shard_range`).
  * One long sequence: rank r owns a contiguous run of pages (`split_pages`), the last rank also owns
    the fp16 window; every rank produces the un-normalised state (max, sum, accumulator) of its part
    and ONE small all-gather (heads x 130 floats per rank) precedes the merge, which is bmx's split
    merge formula applied across ranks (bmx: src/bmx/cache/triton_dequant_attention.py:409-461).
Every kernel reads only its own GPU's memory; the gathered partials land in a local buffer first.
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


class SequenceSplitDecoder:
    """Decode step of one long sequence whose committed pages are split across the ranks of `group`.

    `state` is this rank's layer state (k2b or spectral) holding ITS pages only (and the window on the last rank);
    `first_page` is the index of its first page in the whole sequence, which fixes the rotary positions.
    """

    def __init__(self, state, first_page: int, group=None):
        self.state, self.first_page, self.group = state, first_page, group
        rows = state.batch * state.geom.h_kv * (getattr(state, "n_q_groups", None) or state.geom.n_q_groups)
        self.part = torch.empty(rows, PART_STRIDE, dtype=torch.float32, device=state.device)

    def decode(self, q: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        from . import kernels as K

        st = self.state  # a K2bLayerState or a SpectralLayerState: same call
        st.decode(q, partial_out=self.part, pos_offset=self.first_page * st.page)
        gathered = gather_partials(self.part, self.group)
        return K.merge_partials(gathered, out=out)
