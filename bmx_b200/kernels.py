"""Thin torch-facing wrappers over the bmxk C ABI (include/bmxk.h).

torch is used for device memory and streams only; every function here passes raw pointers to
libbmxk.so and raises `BmxkError` on a non-zero status.  Nothing in this module computes on the CPU.
"""

from __future__ import annotations

import ctypes
import functools
import struct

import torch

from . import _lib
from ._lib import DTYPE_BF16, DTYPE_F16, DTYPE_F32, K2bGeom, call

HEAD_DIM = 128

# Lloyd-Max levels for N(0,1) exactly as bmx computes them at run time
# (bmx: src/bmx/cache/codecs.py:346-380, 2**18 seeded samples, 40 iterations; float32).
GAUSSIAN_CODEBOOK = {
    2: (-1.5194618701934814, -0.46033763885498047, 0.44421979784965515, 1.5017313957214355),
    3: (-2.174412250518799, -1.3567343950271606, -0.7671520113945007, -0.2563295364379883,
        0.23005320131778717, 0.7372721433639526, 1.3183449506759644, 2.12149977684021),
}


@functools.lru_cache(maxsize=16)
def hadamard_signs(d: int, seed: int) -> torch.Tensor:
    """+-1 vector of the randomized Hadamard rotation (bmx: src/bmx/cache/codecs.py:114-124)."""
    g = torch.Generator().manual_seed(seed)
    return (torch.randint(0, 2, (d,), generator=g) * 2 - 1).to(torch.float32)


def _dtype_code(t: torch.Tensor) -> int:
    if t.dtype == torch.float16:
        return DTYPE_F16
    if t.dtype == torch.bfloat16:
        return DTYPE_BF16
    if t.dtype == torch.float32:
        return DTYPE_F32
    raise TypeError(f"unsupported dtype {t.dtype}")


def _ptr(t: torch.Tensor | None):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """Handle of torch's current stream on the current device (the raw getter skips building a Stream object,
    which costs more than a kernel launch)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _require_cuda(*ts: torch.Tensor) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("bmxk kernels take CUDA tensors; there is no CPU path")


def _require_device_visible(*ts: torch.Tensor) -> None:
    """CUDA tensors, or pinned host tensors (mapped into the device's address space: a kernel can read / write them)."""
    for t in ts:
        if t is not None and not (t.is_cuda or t.is_pinned()):
            raise RuntimeError("this argument must be a CUDA tensor or a pinned host tensor")


DEFAULT_K2B_LAYOUT = 1  # row order, read by the tcgen05 decode kernel


def k2b_geom(h_kv: int, n_q_groups: int, page: int = 128, rank: int = 16, group: int = 64,
             n_coef_heads: int = 1, kbits: int = 3, vbits: int = 2, layout: int | None = None) -> K2bGeom:
    """`layout` picks the byte order inside a page block and with it the decode kernel: 1 (row order, tcgen05
    kernel) needs page 128; 0 (fragment order, mma.sync kernel) takes page 64 or 128.  None picks 1 where it fits."""
    if layout is None:
        layout = DEFAULT_K2B_LAYOUT if page == 128 else 0
    return K2bGeom(h_kv, n_q_groups, page, rank, group, n_coef_heads, kbits, vbits, layout)


def page_block_bytes(g: K2bGeom) -> int:
    return int(_lib.lib().bmxk_k2b_page_block_bytes(ctypes.byref(g)))


def coef_block_bytes(g: K2bGeom) -> int:
    return int(_lib.lib().bmxk_k2b_coef_block_bytes(ctypes.byref(g)))


class K2bPool:
    """Device page pool of one layer: `pages[n_slots][h_kv][block]` and `coefs[n_slots][n_coef_heads][block]`."""

    def __init__(self, g: K2bGeom, n_slots: int, device):
        self.geom = g
        self.n_slots = n_slots
        self.pages = torch.zeros(n_slots, g.h_kv, page_block_bytes(g), dtype=torch.uint8, device=device)
        self.coefs = torch.zeros(n_slots, g.n_coef_heads, coef_block_bytes(g), dtype=torch.uint8, device=device)

    def nbytes(self) -> int:
        return self.pages.numel() + self.coefs.numel()


def pack_u(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """bmx pack_codes on the GPU: int16 (rows, C) -> uint8 (rows, C*bits/8)."""
    _require_cuda(codes)
    codes = codes.to(torch.int16).contiguous()
    rows, C = codes.reshape(-1, codes.shape[-1]).shape if codes.numel() else (0, codes.shape[-1])
    if bits not in (2, 4) or C % (8 // max(bits, 1)) != 0:
        call("bmxk_pack_u", _ptr(codes), None, rows, C, bits, _stream())  # raises with the library's message
    out = torch.empty(*codes.shape[:-1], C * bits // 8, dtype=torch.uint8, device=codes.device)
    call("bmxk_pack_u", _ptr(codes), _ptr(out), rows, C, bits, _stream())
    return out


def unpack_u(packed: torch.Tensor, bits: int, C: int) -> torch.Tensor:
    _require_cuda(packed)
    packed = packed.contiguous()
    rows = packed.numel() // max(packed.shape[-1], 1)
    out = torch.empty(*packed.shape[:-1], C, dtype=torch.int16, device=packed.device)
    call("bmxk_unpack_u", _ptr(packed), _ptr(out), rows, C, bits, _stream())
    return out


def pack_s4(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """bmx pack_signed_codes on the GPU: int8 (rows, N) -> uint8 (rows, N/2)."""
    _require_cuda(codes)
    codes = codes.to(torch.int8).contiguous()
    N = codes.shape[-1]
    rows = codes.numel() // max(N, 1)
    if N % 2 or not 1 <= bits <= 4:
        call("bmxk_pack_s4", _ptr(codes), None, rows, N, bits, _stream())
    out = torch.empty(*codes.shape[:-1], N // 2, dtype=torch.uint8, device=codes.device)
    call("bmxk_pack_s4", _ptr(codes), _ptr(out), rows, N, bits, _stream())
    return out


def unpack_s4(packed: torch.Tensor, bits: int, N: int) -> torch.Tensor:
    _require_cuda(packed)
    packed = packed.contiguous()
    rows = packed.numel() // max(packed.shape[-1], 1)
    out = torch.empty(*packed.shape[:-1], N, dtype=torch.int8, device=packed.device)
    call("bmxk_unpack_s4", _ptr(packed), _ptr(out), rows, N, bits, _stream())
    return out


def k2b_append(pool: K2bPool, k_pre: torch.Tensor, v: torch.Tensor, basis_f32: torch.Tensor,
               signs: torch.Tensor, codebook: torch.Tensor, slots: torch.Tensor, n_pages: int) -> None:
    """Quantizes `n_pages` full pages of every sequence in k_pre/v (n_seq, h_kv, T, 128) into the pool.

    slots: int32 (n_seq * n_pages,) physical slot per page, sequence-major.
    """
    g = pool.geom
    _require_cuda(k_pre, v, basis_f32, signs, codebook, slots)
    assert k_pre.shape == v.shape and k_pre.dim() == 4 and k_pre.shape[1] == g.h_kv and k_pre.shape[3] == HEAD_DIM
    assert k_pre.dtype == v.dtype and k_pre.stride() == v.stride() and k_pre.stride(3) == 1
    assert k_pre.shape[2] >= n_pages * g.page
    n_seq = k_pre.shape[0]
    assert slots.dtype == torch.int32 and slots.numel() == n_seq * n_pages
    assert basis_f32.dtype == torch.float32 and basis_f32.shape == (g.h_kv * HEAD_DIM, g.rank) and basis_f32.is_contiguous()
    call("bmxk_k2b_append", ctypes.byref(g), _ptr(k_pre), _ptr(v), _dtype_code(k_pre), k_pre.stride(0), k_pre.stride(1),
         k_pre.stride(2), _ptr(basis_f32), _ptr(signs), _ptr(codebook), _ptr(slots), n_seq, n_pages,
         _ptr(pool.pages), _ptr(pool.coefs), _stream())


def k2b_append_coefs(pool: K2bPool, k_pre: torch.Tensor, v: torch.Tensor, us_f32: torch.Tensor, basis_f32: torch.Tensor,
                     signs: torch.Tensor, codebook: torch.Tensor, slots: torch.Tensor, n_pages: int) -> None:
    """k2b_append with the projection given: us_f32 (n_seq, n_pages * page, rank) float32 = keys of ALL heads of a basis
    spanning all heads, projected (e.g. summed over the ranks that hold the other heads); basis_f32: the basis rows of this
    pool's h_kv heads.  The pool's geometry must have n_coef_heads == 1."""
    g = pool.geom
    _require_cuda(k_pre, v, us_f32, basis_f32, signs, codebook, slots)
    assert g.n_coef_heads == 1, "given coefficients belong to one basis over all heads"
    assert k_pre.shape == v.shape and k_pre.dim() == 4 and k_pre.shape[1] == g.h_kv and k_pre.shape[3] == HEAD_DIM
    assert k_pre.dtype == v.dtype and k_pre.stride() == v.stride() and k_pre.stride(3) == 1
    n_seq = k_pre.shape[0]
    assert k_pre.shape[2] >= n_pages * g.page and slots.dtype == torch.int32 and slots.numel() == n_seq * n_pages
    assert us_f32.dtype == torch.float32 and us_f32.shape == (n_seq, n_pages * g.page, g.rank) and us_f32.is_contiguous()
    assert basis_f32.dtype == torch.float32 and basis_f32.shape == (g.h_kv * HEAD_DIM, g.rank) and basis_f32.is_contiguous()
    call("bmxk_k2b_append_coefs", ctypes.byref(g), _ptr(k_pre), _ptr(v), _dtype_code(k_pre), k_pre.stride(0), k_pre.stride(1),
         k_pre.stride(2), _ptr(us_f32), _ptr(basis_f32), _ptr(signs), _ptr(codebook), _ptr(slots), n_seq, n_pages,
         _ptr(pool.pages), _ptr(pool.coefs), _stream())


def k2b_export_stacks(pool: K2bPool, slots: torch.Tensor) -> dict:
    """Pages -> the tensors bmx's build_kv_stacked_k2b(pack_k=True, pack_v=True) would hold."""
    g = pool.geom
    n, dev, C = slots.numel(), pool.pages.device, g.h_kv * HEAD_DIM
    out = {
        "us": torch.empty(n, g.n_coef_heads, g.page, g.rank, dtype=torch.float16, device=dev),
        "res_int_packed": torch.empty(n, C, g.page // 2, dtype=torch.uint8, device=dev),
        "res_scale": torch.empty(n, C, g.page // g.group, dtype=torch.float16, device=dev),
        "v_idx_packed": torch.empty(n, g.page, C // 4, dtype=torch.uint8, device=dev),
        "v_norm": torch.empty(n, g.page, g.h_kv, dtype=torch.float16, device=dev),
    }
    call("bmxk_k2b_export_stacks", ctypes.byref(g), _ptr(pool.pages), _ptr(pool.coefs), _ptr(slots), n, _ptr(out["us"]),
         _ptr(out["res_int_packed"]), _ptr(out["res_scale"]), _ptr(out["v_idx_packed"]), _ptr(out["v_norm"]), _stream())
    return out


def k2b_dequant_pages(pool: K2bPool, slots: torch.Tensor, basis_f16: torch.Tensor, signs: torch.Tensor,
                      codebook: torch.Tensor, want_k: bool = True, want_v: bool = True):
    """Pages -> float32 (n, page, h_kv*128) pre-RoPE keys and values (bmx dequant_packed)."""
    g = pool.geom
    n, dev, C = slots.numel(), pool.pages.device, g.h_kv * HEAD_DIM
    k = torch.empty(n, g.page, C, dtype=torch.float32, device=dev) if want_k else None
    v = torch.empty(n, g.page, C, dtype=torch.float32, device=dev) if want_v else None
    call("bmxk_k2b_dequant_pages", ctypes.byref(g), _ptr(pool.pages), _ptr(pool.coefs), _ptr(basis_f16), _ptr(signs),
         _ptr(codebook), _ptr(slots), n, _ptr(k), _ptr(v), _stream())
    return k, v


def k2b_dequant_dense(pool: K2bPool, page_table: torch.Tensor, n_pages: int, basis_f16: torch.Tensor, signs: torch.Tensor,
                      codebook: torch.Tensor, rope_cos: torch.Tensor | None, rope_sin: torch.Tensor | None, k_out: torch.Tensor,
                      v_out: torch.Tensor, pos_offset: int = 0) -> None:
    """The first n_pages pages of every sequence -> rotated keys and values in k_out / v_out (batch, h_kv, rows, 128), fp16
    or bf16, rows 0 .. n_pages*page - 1; the rest of the rows is the caller's (the fp16 window)."""
    g = pool.geom
    _require_cuda(page_table, k_out, v_out)
    batch = page_table.shape[0]
    assert page_table.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1
    assert k_out.shape == v_out.shape and k_out.shape[:2] == (batch, g.h_kv) and k_out.shape[3] == HEAD_DIM
    assert k_out.is_contiguous() and v_out.is_contiguous() and k_out.dtype == v_out.dtype
    assert k_out.dtype in (torch.float16, torch.bfloat16), k_out.dtype
    assert rope_cos is None or (rope_cos.dtype == torch.float16 and rope_sin.dtype == torch.float16)
    call("bmxk_k2b_dequant_dense", ctypes.byref(g), _ptr(pool.pages), _ptr(pool.coefs), _ptr(basis_f16), _ptr(signs), _ptr(codebook),
         _ptr(page_table), page_table.stride(0), int(n_pages), batch, _ptr(rope_cos), _ptr(rope_sin), int(pos_offset), _ptr(k_out),
         _ptr(v_out), k_out.shape[2], DTYPE_BF16 if k_out.dtype == torch.bfloat16 else DTYPE_F16, _stream())


@functools.lru_cache(maxsize=8)
def make_v_lut(codebook: tuple) -> tuple:
    """(lo bytes, hi bytes, alpha bits, beta bits) of the fp16 value-level table for `codebook`."""
    cb = (ctypes.c_float * 4)(*codebook)
    out = (ctypes.c_uint32 * 4)()
    call("bmxk_k2b_make_v_lut", cb, out)
    return tuple(int(x) for x in out)


def decode_workspace(g: K2bGeom, batch: int, max_pages: int, device) -> torch.Tensor:
    """Zero-initialised workspace for k2b_decode (status word + per-CTA partial states)."""
    n = int(_lib.lib().bmxk_k2b_decode_workspace_bytes(ctypes.byref(g), batch, max_pages))
    return torch.zeros(n, dtype=torch.uint8, device=device)


def k2b_decode(pool: K2bPool, q: torch.Tensor, basis_f16: torch.Tensor, page_table: torch.Tensor,
               n_pages: torch.Tensor, max_pages: int, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
               k_tail: torch.Tensor | None, v_tail: torch.Tensor | None, tail_len: torch.Tensor | None,
               v_lut_dev: torch.Tensor, signs: torch.Tensor, sm_scale: float, workspace: torch.Tensor,
               out: torch.Tensor | None = None, partial_out: torch.Tensor | None = None,
               pos_offset: int = 0, phases: int = 3) -> torch.Tensor:
    """One decode step for q (batch, heads, 128) fp16 over the paged k2b cache plus the fp16 window."""
    g = pool.geom
    _require_cuda(q, page_table, n_pages, workspace)
    _require_device_visible(out)  # a pinned host tensor: the merge kernel stores the result there itself
    batch = q.shape[0]
    assert q.dtype == torch.float16 and q.is_contiguous() and q.shape[1:] == (g.h_kv * g.n_q_groups, HEAD_DIM)
    assert page_table.dtype == torch.int32 and n_pages.dtype == torch.int32 and page_table.dim() == 2
    tail_cap = 0 if k_tail is None else k_tail.shape[2]
    if k_tail is not None:
        assert k_tail.dtype == torch.float16 and k_tail.is_contiguous() and v_tail.is_contiguous()
        assert k_tail.shape == (batch, g.h_kv, tail_cap, HEAD_DIM) == v_tail.shape
    if out is None and partial_out is None:
        out = torch.empty(batch, g.h_kv * g.n_q_groups, HEAD_DIM, dtype=torch.float16, device=q.device)
    out_code = DTYPE_F16 if out is None else _dtype_code(out)
    call("bmxk_k2b_decode", ctypes.byref(g), _ptr(q), _ptr(pool.pages), _ptr(pool.coefs), _ptr(basis_f16),
         _ptr(page_table), page_table.stride(0), _ptr(n_pages), batch, max_pages, _ptr(rope_cos), _ptr(rope_sin),
         pos_offset, _ptr(k_tail), _ptr(v_tail), _ptr(tail_len), tail_cap, _ptr(v_lut_dev), _ptr(signs),
         ctypes.c_float(sm_scale), _ptr(workspace), workspace.numel(), _ptr(out), out_code, _ptr(partial_out), phases, _stream())
    return out if partial_out is None else partial_out


def k2b_prefill(pool: K2bPool, q: torch.Tensor, q_pos0: int, basis_f16: torch.Tensor, page_table: torch.Tensor, n_pages: torch.Tensor,
                rope_cos: torch.Tensor, rope_sin: torch.Tensor, k_tail: torch.Tensor | None, v_tail: torch.Tensor | None,
                tail_len: torch.Tensor | None, v_lut_dev: torch.Tensor, signs: torch.Tensor, sm_scale: float, status: torch.Tensor,
                out: torch.Tensor | None = None, pos_offset: int = 0, n_split: int = 1) -> torch.Tensor:
    """Causal attention of q (batch, heads, n_q, 128) fp16, rows at positions q_pos0 .. q_pos0 + n_q - 1, over the paged k2b
    cache and the fp16 window, page by page in shared memory (no dense K / V).  status: zeroed device int32 (>= 4).
    n_split > 1 shares the pages of every block of query positions out over that many CTAs (few rows, long context)."""
    g = pool.geom
    _require_cuda(q, page_table, n_pages, status)
    batch, heads, n_q = q.shape[0], q.shape[1], q.shape[2]
    assert q.dtype == torch.float16 and q.is_contiguous() and heads == g.h_kv * g.n_q_groups and q.shape[3] == HEAD_DIM
    assert page_table.dtype == torch.int32 and n_pages.dtype == torch.int32 and status.dtype == torch.int32 and status.numel() >= 4
    tail_cap = 0 if k_tail is None else k_tail.shape[2]
    if k_tail is not None:
        assert k_tail.dtype == torch.float16 and k_tail.is_contiguous() and v_tail.is_contiguous()
        assert k_tail.shape == (batch, g.h_kv, tail_cap, HEAD_DIM) == v_tail.shape
    if out is None:
        out = torch.empty_like(q)
    assert out.dtype == torch.float16 and out.is_contiguous() and out.shape == q.shape
    args = (ctypes.byref(g), _ptr(q), n_q, int(q_pos0), _ptr(pool.pages), _ptr(pool.coefs), _ptr(basis_f16),
            _ptr(page_table), page_table.stride(0), _ptr(n_pages), batch, _ptr(rope_cos), _ptr(rope_sin), int(pos_offset), _ptr(k_tail),
            _ptr(v_tail), _ptr(tail_len), tail_cap, _ptr(v_lut_dev), _ptr(signs), ctypes.c_float(sm_scale), _ptr(status), _ptr(out))
    if n_split <= 1:
        call("bmxk_k2b_prefill", *args, _stream())
        return out
    nbytes = int(_lib.lib().bmxk_k2b_prefill_workspace_bytes(ctypes.byref(g), n_q, batch, int(n_split)))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device)  # the caching allocator keeps it alive until the stream is through
    call("bmxk_k2b_prefill_split", *args, int(n_split), _ptr(ws), nbytes, _stream())
    return out


def k2b_prefill_select(kernel: int) -> None:
    """Process-wide choice of the paged-prefill kernel: 0 = tcgen05 where it applies (default), 1 = mma.sync."""
    call("bmxk_k2b_prefill_select", int(kernel))


STATIC_SCRATCH_BYTES = 2 * 1024 * 1024


def k2b_decode_static(pool: K2bPool, q: torch.Tensor, basis_f16: torch.Tensor, page_table: torch.Tensor,
                      n_pages: torch.Tensor, max_pages: int, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
                      k_tail: torch.Tensor | None, v_tail: torch.Tensor | None, tail_len: torch.Tensor | None,
                      v_lut: torch.Tensor, signs: torch.Tensor, sm_scale: float, out: torch.Tensor,
                      pos_offset: int = 0) -> torch.Tensor:
    """k2b_decode for callers that may not allocate device memory: no workspace argument, the library's
    built-in 2 MiB scratch is used (one per GPU, shared by all calls: do not overlap calls on a GPU).
    Raises BmxkError if the batch needs more scratch than that."""
    g = pool.geom
    _require_cuda(q, page_table, n_pages, out)
    batch = q.shape[0]
    assert q.dtype == torch.float16 and q.is_contiguous() and q.shape[1:] == (g.h_kv * g.n_q_groups, HEAD_DIM)
    tail_cap = 0 if k_tail is None else k_tail.shape[2]
    call("bmxk_k2b_decode_static", ctypes.byref(g), _ptr(q), _ptr(pool.pages), _ptr(pool.coefs), _ptr(basis_f16),
         _ptr(page_table), page_table.stride(0), _ptr(n_pages), batch, max_pages, _ptr(rope_cos), _ptr(rope_sin),
         pos_offset, _ptr(k_tail), _ptr(v_tail), _ptr(tail_len), tail_cap, _ptr(v_lut), _ptr(signs),
         ctypes.c_float(sm_scale), _ptr(out), _dtype_code(out), _stream())
    return out


def k2b_decode_static_status() -> None:
    """Raises BmxkError if a bounded wait of the last k2b_decode_static call on the current device ran out
    (synchronises the current stream; allocates nothing)."""
    call("bmxk_k2b_decode_static_status", _stream())


def selftest_bounded_wait(status: torch.Tensor, limit_cycles: int) -> None:
    """Launches the one-warp kernel that waits on a barrier nobody arrives on; status: zeroed device int32[4]."""
    _require_cuda(status)
    assert status.dtype == torch.int32 and status.numel() >= 4
    call("bmxk_selftest_bounded_wait", _ptr(status), int(limit_cycles), _stream())


def _same_token_layout(x: torch.Tensor, ref: torch.Tensor) -> bool:
    """(batch, h_kv, 1, 128) sources: same dtype, unit channel stride, and equal strides wherever a stride matters
    (a dimension of size one may carry any stride)."""
    return (x.shape == ref.shape and x.dtype == ref.dtype and x.stride(3) == 1 and
            all(x.shape[d] == 1 or x.stride(d) == ref.stride(d) for d in (0, 1)))


def window_append(k_post: torch.Tensor, v: torch.Tensor, k_src: torch.Tensor, k_win: torch.Tensor, v_win: torch.Tensor,
                  k_src_win: torch.Tensor, tail_len: torch.Tensor, t: int) -> None:
    """One new token per sequence, (batch, h_kv, 1, 128) each, into position t of the fp16 windows; one launch."""
    _require_cuda(k_post, v, k_src, k_win, v_win, k_src_win, tail_len)
    batch, h_kv = k_post.shape[0], k_post.shape[1]
    srcs = [k_post, v, k_src]
    if any(x.shape[2] != 1 or x.shape[3] != 128 for x in srcs):
        raise ValueError("window_append: sources must be (batch, h_kv, 1, 128)")
    if not all(_same_token_layout(x, k_post) for x in srcs):
        srcs = [x.to(k_post.dtype).contiguous() for x in srcs]  # a few KB: one common layout for the kernel
    k_post, v, k_src = srcs
    call("bmxk_window_append", _ptr(k_post), _ptr(v), _ptr(k_src), _dtype_code(k_post), k_post.stride(0), k_post.stride(1),
         _ptr(k_win), _ptr(v_win), _ptr(k_src_win), _ptr(tail_len), batch, h_kv, k_win.shape[2], int(t), _stream())


def window_append_devpos(k_post: torch.Tensor, v: torch.Tensor, k_src: torch.Tensor, k_win: torch.Tensor, v_win: torch.Tensor,
                         k_src_win: torch.Tensor, tail_len: torch.Tensor, counters: torch.Tensor,
                         status: torch.Tensor | None = None) -> None:
    """window_append at the position held in tail_len (device int32 per sequence), which the kernel advances: no
    per-step argument, so the launch can sit in a CUDA graph.  Sources: (batch, h_kv, 1, 128), one dtype and layout.
    counters: device int32 (batch), zero-initialised once and owned by these calls."""
    _require_cuda(k_post, v, k_src, k_win, v_win, k_src_win, tail_len, counters)
    assert counters.dtype == torch.int32 and counters.numel() >= k_post.shape[0]
    batch, h_kv = k_post.shape[0], k_post.shape[1]
    for x in (k_post, v, k_src):
        if not _same_token_layout(x, k_post):
            raise ValueError("window_append_devpos: sources must share shape (batch, h_kv, 1, 128), dtype and strides")
    call("bmxk_window_append_devpos", _ptr(k_post), _ptr(v), _ptr(k_src), _dtype_code(k_post), k_post.stride(0), k_post.stride(1),
         _ptr(k_win), _ptr(v_win), _ptr(k_src_win), _ptr(tail_len), _ptr(counters), _ptr(status), batch, h_kv, k_win.shape[2],
         _stream())


def gather_next_slots(page_table: torch.Tensor, n_pages: torch.Tensor, n: int, out: torch.Tensor) -> torch.Tensor:
    """out[s * n + i] = page_table[s, n_pages[s] + i] (device-side lookup of the next n pages' slots of every sequence)."""
    _require_cuda(page_table, n_pages, out)
    assert page_table.dtype == n_pages.dtype == out.dtype == torch.int32 and page_table.dim() == 2 and page_table.stride(1) == 1
    batch = page_table.shape[0]
    assert out.numel() >= batch * n and out.is_contiguous()
    call("bmxk_gather_next_slots", _ptr(page_table), page_table.stride(0), _ptr(n_pages), batch, int(n), _ptr(out), _stream())
    return out


def window_shift(k_win: torch.Tensor, v_win: torch.Tensor, k_src_win: torch.Tensor, off: int, rest: int, tail_len: torch.Tensor,
                 n_pages: torch.Tensor | None = None, pages_added: int = 0) -> None:
    """Moves tokens [off, off + rest) of every (sequence, head) window to the front (one launch for the three windows),
    sets the device-side window length to rest and adds pages_added to the device-side page counts."""
    _require_cuda(k_win, v_win, k_src_win, tail_len, n_pages)
    assert k_win.is_contiguous() and v_win.is_contiguous() and k_src_win.is_contiguous() and k_win.shape == v_win.shape == k_src_win.shape
    batch, h_kv, tail_cap = k_win.shape[0], k_win.shape[1], k_win.shape[2]
    call("bmxk_window_shift", _ptr(k_win), _ptr(v_win), _ptr(k_src_win), batch, h_kv, tail_cap, int(off), int(rest), _ptr(tail_len),
         _ptr(n_pages), int(pages_added), _stream())


def step_ingest(q_src: torch.Tensor, q_dst: torch.Tensor, k_post: torch.Tensor, v: torch.Tensor, k_src: torch.Tensor,
                k_win: torch.Tensor, v_win: torch.Tensor, k_src_win: torch.Tensor, tail_len: torch.Tensor, counters: torch.Tensor,
                status: torch.Tensor | None = None) -> None:
    """One launch for a decode step's inputs: the token (k_post, v, k_src: (batch, h_kv, 1, 128) fp16) goes into the
    windows at the device-side position, the queries q_src (batch, heads, 128) fp16 are staged into q_dst.  The four
    sources may be pinned host tensors: the kernel then reads them over PCIe and no separate copy is needed."""
    _require_device_visible(q_src, k_post, v, k_src)
    _require_cuda(q_dst, k_win, v_win, k_src_win, tail_len, counters)
    batch, h_kv = k_post.shape[0], k_post.shape[1]
    for x in (k_post, v, k_src):
        if x.dtype != torch.float16 or not _same_token_layout(x, k_post):
            raise ValueError("step_ingest: token sources must be fp16 (batch, h_kv, 1, 128) with one layout")
    assert q_src.dtype == q_dst.dtype == torch.float16 and q_src.shape == q_dst.shape and q_src.is_contiguous() and q_dst.is_contiguous()
    assert q_src.shape[0] == batch and q_src.shape[1] % h_kv == 0 and q_src.shape[2] == HEAD_DIM
    call("bmxk_step_ingest", _ptr(q_src), _ptr(q_dst), q_src.shape[1] // h_kv, _ptr(k_post), _ptr(v), _ptr(k_src), k_post.stride(0),
         k_post.stride(1), _ptr(k_win), _ptr(v_win), _ptr(k_src_win), _ptr(tail_len), _ptr(counters), _ptr(status), batch, h_kv,
         k_win.shape[2], _stream())


def merge_partials(parts: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """(n_parts, rows, 130) float32 partial states -> normalised (rows, 128) output (bmx split merge)."""
    _require_cuda(parts)
    assert parts.dtype == torch.float32 and parts.dim() == 3 and parts.shape[2] == 130 and parts.is_contiguous()
    n, rows = parts.shape[0], parts.shape[1]
    if out is None:
        out = torch.empty(rows, HEAD_DIM, dtype=torch.float16, device=parts.device)
    call("bmxk_merge_partials", _ptr(parts), n, rows, _ptr(out), _dtype_code(out), _stream())
    return out


def v_lut_tensor(codebook: tuple, device) -> torch.Tensor:
    """Host-side copy of the value table, as the int32 tensor whose 4 words bmxk_k2b_decode reads."""
    return torch.tensor([struct.unpack("<i", struct.pack("<I", x))[0] for x in make_v_lut(tuple(codebook))],
                        dtype=torch.int32)


def check_status(workspace: torch.Tensor) -> None:
    call("bmxk_check_workspace_status", _ptr(workspace), _stream())


# ---- plain RTN caches ---------------------------------------------------------------------------

from ._lib import RtnGeom  # noqa: E402

RTN_TOKEN, RTN_CHANNEL = 0, 1


def rtn_geom(h_kv: int, n_q_groups: int, page: int = 128, k_arm: str = "rtn_token", k_group: int = 32,
             v_group: int = 32, kbits: int = 4, vbits: int = 2) -> RtnGeom:
    arm = {"rtn_token": RTN_TOKEN, "rtn_channel": RTN_CHANNEL}[k_arm]
    return RtnGeom(h_kv, n_q_groups, page, arm, k_group, v_group, kbits, vbits)


class RtnPool:
    """Device page pool of one layer of an RTN cache: `pages[n_slots][h_kv][block]`."""

    def __init__(self, g: RtnGeom, n_slots: int, device):
        self.geom, self.n_slots = g, n_slots
        nb = int(_lib.lib().bmxk_rtn_page_block_bytes(ctypes.byref(g)))
        self.pages = torch.zeros(n_slots, g.h_kv, nb, dtype=torch.uint8, device=device)


def rtn_append(pool: RtnPool, k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, n_pages: int) -> None:
    """Quantizes n_pages full pages of every sequence of k/v (n_seq, h_kv, T, 128); keys are post-RoPE."""
    g = pool.geom
    _require_cuda(k, v, slots)
    assert k.shape == v.shape and k.dim() == 4 and k.shape[1] == g.h_kv and k.shape[3] == HEAD_DIM
    assert k.dtype == v.dtype and k.stride() == v.stride() and k.stride(3) == 1 and k.shape[2] >= n_pages * g.page
    assert slots.dtype == torch.int32 and slots.numel() == k.shape[0] * n_pages
    call("bmxk_rtn_append", ctypes.byref(g), _ptr(k), _ptr(v), _dtype_code(k), k.stride(0), k.stride(1), k.stride(2),
         _ptr(slots), k.shape[0], n_pages, _ptr(pool.pages), _stream())


def rtn_export(pool: RtnPool, slots: torch.Tensor, dequant: bool = False) -> dict:
    """Pages -> bmx's int8 code containers and fp16 scales (and, on request, float32 dequantized pages)."""
    g = pool.geom
    n, dev, C = slots.numel(), pool.pages.device, g.h_kv * HEAD_DIM
    if g.k_arm == RTN_TOKEN:
        kc = torch.empty(n, g.h_kv, g.page, HEAD_DIM, dtype=torch.int8, device=dev)
        ks = torch.empty(n, g.h_kv, g.page, HEAD_DIM // g.k_group, dtype=torch.float16, device=dev)
    else:
        kc = torch.empty(n, C, g.page, dtype=torch.int8, device=dev)
        ks = torch.empty(n, C, g.page // g.k_group, dtype=torch.float16, device=dev)
    out = {"k_codes": kc, "k_scales": ks,
           "v_codes": torch.empty(n, g.h_kv, g.page, HEAD_DIM, dtype=torch.int8, device=dev),
           "v_scales": torch.empty(n, g.h_kv, g.page, HEAD_DIM // g.v_group, dtype=torch.float16, device=dev)}
    if dequant:
        out["k_deq"] = torch.empty(n, g.page, C, dtype=torch.float32, device=dev)
        out["v_deq"] = torch.empty(n, g.page, C, dtype=torch.float32, device=dev)
    call("bmxk_rtn_export", ctypes.byref(g), _ptr(pool.pages), _ptr(slots), n, _ptr(kc), _ptr(ks), _ptr(out["v_codes"]),
         _ptr(out["v_scales"]), _ptr(out.get("k_deq")), _ptr(out.get("v_deq")), _stream())
    return out


def rtn_workspace(g: RtnGeom, batch: int, max_pages: int, device) -> torch.Tensor:
    n = int(_lib.lib().bmxk_rtn_decode_workspace_bytes(ctypes.byref(g), batch, max_pages))
    return torch.zeros(n, dtype=torch.uint8, device=device)


def rtn_decode(pool: RtnPool, q: torch.Tensor, page_table: torch.Tensor, n_pages: torch.Tensor, max_pages: int,
               k_tail: torch.Tensor | None, v_tail: torch.Tensor | None, tail_len: torch.Tensor | None,
               sm_scale: float, workspace: torch.Tensor, out: torch.Tensor | None = None,
               partial_out: torch.Tensor | None = None) -> torch.Tensor:
    """One decode step for q (batch, heads, 128) fp16 over RTN pages plus the fp16 window."""
    g = pool.geom
    _require_cuda(q, page_table, n_pages, workspace)
    batch = q.shape[0]
    assert q.dtype == torch.float16 and q.is_contiguous() and q.shape[1:] == (g.h_kv * g.n_q_groups, HEAD_DIM)
    tail_cap = 0 if k_tail is None else k_tail.shape[2]
    if out is None and partial_out is None:
        out = torch.empty(batch, g.h_kv * g.n_q_groups, HEAD_DIM, dtype=torch.float16, device=q.device)
    out_code = DTYPE_F16 if out is None else _dtype_code(out)
    call("bmxk_rtn_decode", ctypes.byref(g), _ptr(q), _ptr(pool.pages), _ptr(page_table), page_table.stride(0),
         _ptr(n_pages), batch, max_pages, _ptr(k_tail), _ptr(v_tail), _ptr(tail_len), tail_cap, ctypes.c_float(sm_scale),
         _ptr(workspace), workspace.numel(), _ptr(out), out_code, _ptr(partial_out), _stream())
    return out if partial_out is None else partial_out


# ---- K4 spectral key codec (per-head packs) -------------------------------------------------------

from ._lib import SpectralGeom  # noqa: E402

SPECTRAL_TIERS = (0, 2, 3, 4, 5, 6, 8)


def _container_bits(b: int) -> int:
    return 0 if b == 0 else (2 if b == 2 else (4 if b <= 4 else 8))


class SpectralPackDev:
    """Device copy of per-head spectral packs plus the page layout derived from their bit widths.

    enc, dec: (h_kv, 128, 128) float32 with Y = M @ enc[h] and M_hat = Y_hat @ dec[h].T; bits: (h_kv, 128)
    integers from SPECTRAL_TIERS (bmx: SpectralPack, src/bmx/cache/spectral.py:174-220, one pack per head)."""

    def __init__(self, enc: torch.Tensor, dec: torch.Tensor, bits: torch.Tensor, page: int, group: int, device):
        h_kv = enc.shape[0]
        assert enc.shape == dec.shape == (h_kv, HEAD_DIM, HEAD_DIM) and bits.shape == (h_kv, HEAD_DIM)
        assert all(int(b) in SPECTRAL_TIERS for b in bits.reshape(-1).tolist()), "bit widths must be tier members"
        col_off = torch.zeros(h_kv, HEAD_DIM, dtype=torch.int32)
        code_bytes = 0
        for h in range(h_kv):
            off = 0
            for b in sorted(set(int(x) for x in bits[h].tolist())):  # directions laid out tier by tier, ascending
                for j in (bits[h] == b).nonzero().flatten().tolist():
                    col_off[h, j] = off
                    off += page * _container_bits(b) // 8
            code_bytes = max(code_bytes, off)
        scale_off = (code_bytes + 15) // 16 * 16
        block = scale_off + HEAD_DIM * (page // group) * 4
        self.geom = SpectralGeom(h_kv, page, group, (block + 15) // 16 * 16, scale_off)
        self.bits = bits.to(torch.int32)
        self.enc = enc.to(device, torch.float32).contiguous()
        self.dec = dec.to(device, torch.float32).contiguous()
        self.col_bits = self.bits.to(device).contiguous()
        self.col_off = col_off.to(device).contiguous()
        self.device = device
        # what the fused decode kernel reads: directions in tier order (those with bits first, by ascending bits, then
        # ascending index; those without last),
        # the decoder with its columns in that order as the fp16 tensor-core operand, and one word per position
        order = torch.stack([torch.tensor(sorted(range(HEAD_DIM), key=lambda j: (int(bits[h, j]) == 0, int(bits[h, j]), j)))
                             for h in range(h_kv)])
        self.order = order
        meta = col_off.gather(1, order) | (order.to(torch.int32) << 16) | (self.bits.gather(1, order) << 24)
        used = (self.bits > 0).sum(1).clamp(min=1)
        meta[:, 0] |= (((used + 15) // 16 - 1).to(torch.int32) << 28)  # K = 16 steps of the decoder product
        self.meta = meta.to(torch.int32).to(device).contiguous()
        self.set_decode_decoder(dec)

    def set_decode_decoder(self, dec: torch.Tensor) -> None:
        """Decoder used by the fused decode kernel, (h_kv, 128, 128) float32 (e.g. the int8 round trip of the
        pack's decoder, bmx: src/bmx/cache/spectral.py:913-943); stored as fp16 with columns in tier order."""
        idx = self.order.unsqueeze(1).expand(-1, HEAD_DIM, -1)
        self.dec16 = dec.to(torch.float32).cpu().gather(2, idx).to(torch.float16).to(self.device).contiguous()

    def new_pool(self, n_slots: int) -> torch.Tensor:
        return torch.zeros(n_slots, self.geom.h_kv, self.geom.block_bytes, dtype=torch.uint8, device=self.device)


def spectral_append(pack: SpectralPackDev, pool: torch.Tensor, k_pre: torch.Tensor, slots: torch.Tensor, n_pages: int) -> None:
    """Encodes and quantizes n_pages pages of every sequence of k_pre (n_seq, h_kv, T, 128) into the pool."""
    _require_cuda(k_pre, slots, pool)
    g = pack.geom
    assert k_pre.dim() == 4 and k_pre.shape[1] == g.h_kv and k_pre.shape[3] == HEAD_DIM and k_pre.stride(3) == 1
    assert slots.dtype == torch.int32 and slots.numel() == k_pre.shape[0] * n_pages
    call("bmxk_spectral_append", ctypes.byref(g), _ptr(k_pre), _dtype_code(k_pre), k_pre.stride(0), k_pre.stride(1),
         k_pre.stride(2), _ptr(pack.enc), _ptr(pack.col_bits), _ptr(pack.col_off), _ptr(slots), k_pre.shape[0], n_pages,
         _ptr(pool), _stream())


def spectral_dequant_pages(pack: SpectralPackDev, pool: torch.Tensor, slots: torch.Tensor, want_codes: bool = True,
                           want_k: bool = True) -> dict:
    """Pages -> {"codes": int8 (n, h, 128, page), "scales": float32 (n, h, 128, page/group), "k": float32 (n, page, h*128)}."""
    g, n, dev = pack.geom, slots.numel(), pool.device
    out = {}
    if want_codes:
        out["codes"] = torch.empty(n, g.h_kv, HEAD_DIM, g.page, dtype=torch.int8, device=dev)
        out["scales"] = torch.empty(n, g.h_kv, HEAD_DIM, g.page // g.group, dtype=torch.float32, device=dev)
    if want_k:
        out["k"] = torch.empty(n, g.page, g.h_kv * HEAD_DIM, dtype=torch.float32, device=dev)
    call("bmxk_spectral_dequant_pages", ctypes.byref(g), _ptr(pool), _ptr(pack.dec), _ptr(pack.col_bits), _ptr(pack.col_off),
         _ptr(slots), n, _ptr(out.get("codes")), _ptr(out.get("scales")), _ptr(out.get("k")), _stream())
    return out


def spectral_tier_dict(pack: SpectralPackDev, codes: torch.Tensor, scales: torch.Tensor, head: int) -> dict:
    """bmx's flat packed dict {t{b}_codes, t{b}_scale} of one page and head from unpacked codes (128, page)
    and scales (128, page/group): the same containers spectral_quantize_packed returns."""
    out = {}
    bits = pack.bits[head]
    for b in sorted(set(int(x) for x in bits.tolist())):
        if b == 0:
            continue
        cols = (bits == b).nonzero().flatten().to(codes.device)
        q = codes[cols]
        if b in (2, 4):
            out[f"t{b}_codes"] = pack_u((q.to(torch.int16) + 2 ** (b - 1)), b)
        elif b == 3:
            out[f"t{b}_codes"] = pack_s4(q, b)
        else:
            out[f"t{b}_codes"] = q
        out[f"t{b}_scale"] = scales[cols].unsqueeze(-1)
    return out


# ---- value-only page blocks and the fused spectral decode -----------------------------------------


def vblock_pool(h_kv: int, n_slots: int, device) -> torch.Tensor:
    return torch.zeros(n_slots, h_kv, int(_lib.lib().bmxk_vblock_bytes()), dtype=torch.uint8, device=device)


def vblock_append(vpool: torch.Tensor, v: torch.Tensor, signs: torch.Tensor, codebook: torch.Tensor, slots: torch.Tensor,
                  n_pages: int) -> None:
    """Quantizes n_pages 128-token pages of every sequence of v (n_seq, h_kv, T, 128) into value blocks."""
    _require_cuda(vpool, v, signs, codebook, slots)
    h_kv = vpool.shape[1]
    assert v.dim() == 4 and v.shape[1] == h_kv and v.shape[3] == HEAD_DIM and v.stride(3) == 1 and v.shape[2] >= 128 * n_pages
    assert slots.dtype == torch.int32 and slots.numel() == v.shape[0] * n_pages
    call("bmxk_vblock_append", h_kv, _ptr(v), _dtype_code(v), v.stride(0), v.stride(1), v.stride(2), _ptr(signs), _ptr(codebook),
         _ptr(slots), v.shape[0], n_pages, _ptr(vpool), _stream())


def vblock_export(vpool: torch.Tensor, slots: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Value blocks -> bmx's (v_idx_packed uint8 (n, 128, C/4), v_norm fp16 (n, 128, h_kv))."""
    h_kv, n, dev = vpool.shape[1], slots.numel(), vpool.device
    idx = torch.empty(n, 128, h_kv * HEAD_DIM // 4, dtype=torch.uint8, device=dev)
    norm = torch.empty(n, 128, h_kv, dtype=torch.float16, device=dev)
    call("bmxk_vblock_export", h_kv, _ptr(vpool), _ptr(slots), n, _ptr(idx), _ptr(norm), _stream())
    return idx, norm


def spectral_decode_workspace(pack: SpectralPackDev, n_q_groups: int, batch: int) -> torch.Tensor:
    n = int(_lib.lib().bmxk_spectral_decode_workspace_bytes(ctypes.byref(pack.geom), n_q_groups, batch))
    return torch.zeros(n, dtype=torch.uint8, device=pack.device)


def spectral_decode(pack: SpectralPackDev, n_q_groups: int, kpool: torch.Tensor, vpool: torch.Tensor, q: torch.Tensor,
                    page_table: torch.Tensor, n_pages: torch.Tensor, max_pages: int, rope_cos: torch.Tensor,
                    rope_sin: torch.Tensor, k_tail: torch.Tensor | None, v_tail: torch.Tensor | None,
                    tail_len: torch.Tensor | None, v_lut: torch.Tensor, signs: torch.Tensor, sm_scale: float,
                    workspace: torch.Tensor, out: torch.Tensor | None = None, partial_out: torch.Tensor | None = None,
                    pos_offset: int = 0, phases: int = 3) -> torch.Tensor:
    """One decode step for q (batch, heads, 128) fp16 over spectral key pages + value blocks + the fp16 window."""
    g = pack.geom
    _require_cuda(q, kpool, vpool, page_table, n_pages, workspace)
    batch = q.shape[0]
    assert q.dtype == torch.float16 and q.is_contiguous() and q.shape[1:] == (g.h_kv * n_q_groups, HEAD_DIM)
    assert page_table.dtype == torch.int32 and n_pages.dtype == torch.int32 and page_table.dim() == 2
    assert rope_cos.dtype == torch.float16 and rope_sin.dtype == torch.float16
    tail_cap = 0 if k_tail is None else k_tail.shape[2]
    if k_tail is not None:
        assert k_tail.dtype == torch.float16 and k_tail.is_contiguous() and v_tail.is_contiguous()
        assert k_tail.shape == (batch, g.h_kv, tail_cap, HEAD_DIM) == v_tail.shape
    if out is None and partial_out is None:
        out = torch.empty(batch, g.h_kv * n_q_groups, HEAD_DIM, dtype=torch.float16, device=q.device)
    out_code = DTYPE_F16 if out is None else _dtype_code(out)
    call("bmxk_spectral_decode", ctypes.byref(g), n_q_groups, _ptr(q), _ptr(kpool), _ptr(vpool), _ptr(pack.dec16), _ptr(pack.meta),
         _ptr(page_table), page_table.stride(0), _ptr(n_pages), batch, max_pages, _ptr(rope_cos), _ptr(rope_sin), pos_offset,
         _ptr(k_tail), _ptr(v_tail), _ptr(tail_len), tail_cap, _ptr(v_lut), _ptr(signs), ctypes.c_float(sm_scale),
         _ptr(workspace), workspace.numel(), _ptr(out), out_code, _ptr(partial_out), phases, _stream())
    return out if partial_out is None else partial_out
