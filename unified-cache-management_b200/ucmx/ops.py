"""Tensor-level front-end of the C ABI: each function checks shapes, takes raw device pointers
from torch tensors and enqueues the CUDA kernel on torch's current stream.

torch is used for device memory and streams only; all arithmetic happens in libucmx.so.  Nothing
here computes on the CPU and nothing falls back when the library is unavailable.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _native as N
from ._native import (DT_BF16, DT_F32, DT_I32, ORDER_INDEX_ASC, ORDER_SCORE_DESC, POOL_MAX,  # noqa: F401
                      POOL_MEAN, POOL_MIN, POOL_SUM, WIN_EXCLUDE, WIN_FORCE, WIN_NONE)

_POOL_MODES = {"mean": POOL_MEAN, "max": POOL_MAX, "min": POOL_MIN, "sum": POOL_SUM}


def _stream(t: torch.Tensor) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def _exchange(ex):
    """Host pointer to a PeerScoreExchange's ucmx_peer_exchange descriptor (NULL for a single rank)."""
    return None if ex is None else C.byref(ex.desc)


def _need_cuda(*ts: Optional[torch.Tensor]) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("ucmx ops take CUDA tensors; there is no CPU path")


def _i32(t: Optional[torch.Tensor], name: str) -> Optional[torch.Tensor]:
    if t is None:
        return None
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous int32 tensor")
    return t


def kv_geometry(k_cache: torch.Tensor) -> N.KvGeometry:
    """Geometry of a paged cache tensor [num_blocks, block_tokens, n_kv_heads, head_dim] (bf16)."""
    if k_cache.dim() != 4 or k_cache.dtype != torch.bfloat16:
        raise ValueError("k_cache must be bf16 [num_blocks, block_tokens, n_kv_heads, head_dim]")
    nb, T, H, D = k_cache.shape
    sb, st, sh, sd = k_cache.stride()
    if sd != 1 or sh != D:
        raise ValueError("heads and head_dim of the paged cache must be contiguous")
    return N.KvGeometry(sb, st, T, H, D, nb)


def pool_blocks(k_cache: torch.Tensor, block_ids: torch.Tensor, *, mode: str = "mean",
                out_slots: Optional[torch.Tensor] = None, out_bf16: Optional[torch.Tensor] = None,
                out_f32: Optional[torch.Tensor] = None, round_bf16: bool = True, n_rep: int = 1,
                rep_index: int = 0) -> torch.Tensor:
    """Per-block key representatives. Returns the bf16 table (or the fp32 one if only that is given).

    With no output tensor given, a bf16 [n, n_kv_heads, n_rep, head_dim] table is allocated."""
    _need_cuda(k_cache, block_ids, out_slots, out_bf16, out_f32)
    g = kv_geometry(k_cache)
    ids = _i32(block_ids, "block_ids")
    n = ids.numel()
    if out_bf16 is None and out_f32 is None:
        out_bf16 = torch.empty((n, g.n_kv_heads, n_rep, g.head_dim), dtype=torch.bfloat16, device=k_cache.device)
    if out_bf16 is not None and (out_bf16.dtype != torch.bfloat16 or not out_bf16.is_contiguous()):
        raise ValueError("out_bf16 must be contiguous bf16")
    if out_f32 is not None and (out_f32.dtype != torch.float32 or not out_f32.is_contiguous()):
        raise ValueError("out_f32 must be contiguous fp32")
    table = out_bf16 if out_bf16 is not None else out_f32
    rows = table.numel() // (g.n_kv_heads * n_rep * g.head_dim)          # rows of the output table
    st = N.lib.ucmx_pool_blocks(_ptr(k_cache), C.byref(g), _ptr(ids), _ptr(_i32(out_slots, "out_slots")), rows, n,
                                _POOL_MODES[mode], int(round_bf16), n_rep, rep_index, _ptr(out_bf16),
                                _ptr(out_f32), _stream(k_cache))
    N.check("ucmx_pool_blocks", st, 1 if n else 0)
    return out_bf16 if out_bf16 is not None else out_f32


def query_group_mean(query: torch.Tensor, n_kv_heads: int, *, round_bf16: bool = True,
                     out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """query bf16 [n_tok, n_q_heads, head_dim] -> fp32 [n_tok, n_kv_heads*head_dim]."""
    _need_cuda(query, out)
    if query.dim() != 3 or query.dtype != torch.bfloat16:
        raise ValueError("query must be bf16 [n_tok, n_q_heads, head_dim]")
    nt, Hq, D = query.shape
    if query.stride(2) != 1 or query.stride(1) != D:
        query = query.contiguous()
    if out is None:
        out = torch.empty((nt, n_kv_heads * D), dtype=torch.float32, device=query.device)
    st = N.lib.ucmx_query_group_mean(_ptr(query), nt, Hq, n_kv_heads, D, query.stride(0), int(round_bf16),
                                     _ptr(out), _stream(query))
    N.check("ucmx_query_group_mean", st, 1 if nt else 0)
    return out


def score_dot(reps: torch.Tensor, req_offsets: torch.Tensor, q: torch.Tensor, *, total: int,
              slot_ids: Optional[torch.Tensor] = None, n_kv_heads: int, head_dim: int, n_rep: int = 1,
              scale: float = 1.0, out: Optional[torch.Tensor] = None, exchange=None, early: bool = False) -> torch.Tensor:
    """Ragged query-to-block dot scores. reps: bf16 or fp32 table [slots, n_kv_heads, n_rep, head_dim]
    (any shape with that memory layout); q fp32 [n_req, n_kv_heads*head_dim]. Returns fp32 [total].
    exchange: a parallel.PeerScoreExchange under tensor parallelism; the scores then also go to every rank's inbox.
    early: the kernel may begin before the kernel ahead of it in the stream has ended (ucmx_set_early_start); the
    caller vouches that reps, req_offsets, slot_ids and q are not outputs of that kernel."""
    _need_cuda(reps, req_offsets, q, slot_ids, out)
    if reps.dtype == torch.bfloat16:
        dt = DT_BF16
    elif reps.dtype == torch.float32:
        dt = DT_F32
    else:
        raise ValueError("reps must be bf16 or fp32")
    if not reps.is_contiguous() or q.dtype != torch.float32 or not q.is_contiguous():
        raise ValueError("reps and q must be contiguous; q must be fp32")
    n_req = req_offsets.numel() - 1
    if q.numel() != n_req * n_kv_heads * head_dim:
        raise ValueError("q must hold n_req rows of n_kv_heads*head_dim values")
    if out is None and exchange is None:
        out = torch.empty((total,), dtype=torch.float32, device=reps.device)
    n_slots = reps.numel() // (n_kv_heads * n_rep * head_dim)
    if early:
        N.lib.ucmx_set_early_start(1)
    try:
        st = N.lib.ucmx_score_dot(_ptr(reps), dt, n_slots, n_kv_heads, n_rep, head_dim, _ptr(_i32(req_offsets, "req_offsets")),
                                  _ptr(_i32(slot_ids, "slot_ids")), _ptr(q), n_req, total, float(scale), _ptr(out),
                                  _exchange(exchange), _stream(reps))
    finally:
        if early:
            N.lib.ucmx_set_early_start(0)
    N.check("ucmx_score_dot", st, 1 if total and n_req else 0)
    return out


def score_dot_query(reps: torch.Tensor, req_offsets: torch.Tensor, query: torch.Tensor, *, total: int,
                    slot_ids: Optional[torch.Tensor] = None, n_kv_heads: int, round_bf16: bool = True,
                    scale: float = 1.0, out: Optional[torch.Tensor] = None, exchange=None,
                    early: bool = False) -> torch.Tensor:
    """score_dot with the per-KV-head query mean folded in: query is the raw bf16 [n_req, n_q_heads, head_dim].
    Shapes the single-pass kernel does not cover go through query_group_mean + score_dot (two launches).
    early: the kernel may begin before the kernel ahead of it in the stream has ended (ucmx_set_early_start); the
    caller vouches that reps, req_offsets, slot_ids and query are not outputs of that kernel."""
    _need_cuda(reps, req_offsets, query, slot_ids, out)
    if query.dim() != 3 or query.dtype != torch.bfloat16:
        raise ValueError("query must be bf16 [n_req, n_q_heads, head_dim]")
    n_req, Hq, D = query.shape
    if n_req != req_offsets.numel() - 1:
        raise ValueError("one query row per request")
    if query.stride(2) != 1 or query.stride(1) != D:
        query = query.contiguous()
    dt = DT_BF16 if reps.dtype == torch.bfloat16 else DT_F32 if reps.dtype == torch.float32 else None
    if dt is None or not reps.is_contiguous():
        raise ValueError("reps must be contiguous bf16 or fp32")
    if out is None and exchange is None:
        out = torch.empty((total,), dtype=torch.float32, device=reps.device)
    n_slots = reps.numel() // (n_kv_heads * D)
    if early:
        N.lib.ucmx_set_early_start(1)
    try:
        st = N.lib.ucmx_score_dot_query(_ptr(reps), dt, n_slots, n_kv_heads, D, _ptr(_i32(req_offsets, "req_offsets")),
                                        _ptr(_i32(slot_ids, "slot_ids")), _ptr(query), Hq, query.stride(0), int(round_bf16),
                                        n_req, total, float(scale), _ptr(out), _exchange(exchange), _stream(reps))
    finally:
        if early:
            N.lib.ucmx_set_early_start(0)
    if st == N.EUNSUPPORTED:
        qbar = query_group_mean(query, n_kv_heads, round_bf16=round_bf16)
        return score_dot(reps, req_offsets, qbar, total=total, slot_ids=slot_ids, n_kv_heads=n_kv_heads, head_dim=D,
                         scale=scale, out=out, exchange=exchange)
    N.check("ucmx_score_dot_query", st, 1 if total and n_req else 0)
    return out


def score_dot_heads(reps: torch.Tensor, req_offsets: torch.Tensor, query: torch.Tensor, *, total: int,
                    slot_ids: Optional[torch.Tensor] = None, include_mask: Optional[torch.Tensor] = None,
                    exclude_mask: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """GSA's device-side block weights: mean over query heads of the per-head maximum over a block's
    representatives.  reps bf16 [n_slots, H, n_rep, D]; query bf16 [n_req, Hq, D]; masks uint8 [total]."""
    _need_cuda(reps, req_offsets, query, slot_ids, include_mask, exclude_mask, out)
    if reps.dim() != 4 or reps.dtype != torch.bfloat16 or not reps.is_contiguous():
        raise ValueError("reps must be contiguous bf16 [n_slots, n_kv_heads, n_rep, head_dim]")
    if query.dim() != 3 or query.dtype != torch.bfloat16 or query.stride(2) != 1 or query.stride(1) != query.shape[2]:
        raise ValueError("query must be bf16 [n_req, n_q_heads, head_dim] with contiguous heads")
    for m in (include_mask, exclude_mask):
        if m is not None and (m.dtype != torch.uint8 or not m.is_contiguous() or m.numel() != total):
            raise ValueError("masks must be contiguous uint8 [total]")
    n_slots, H, R, D = reps.shape
    n_req = req_offsets.numel() - 1
    if out is None:
        out = torch.empty((total,), dtype=torch.float32, device=reps.device)
    st = N.lib.ucmx_score_dot_heads(_ptr(reps), n_slots, H, R, D, _ptr(_i32(req_offsets, "req_offsets")), _ptr(_i32(slot_ids, "slot_ids")),
                                    _ptr(query), query.shape[1], query.stride(0), n_req, total, _ptr(include_mask),
                                    _ptr(exclude_mask), _ptr(out), _stream(reps))
    N.check("ucmx_score_dot_heads", st, 1 if total and n_req else 0)
    return out


def score_hamming(codes: torch.Tensor, req_offsets: torch.Tensor, q_codes: torch.Tensor, *, total: int,
                  slot_ids: Optional[torch.Tensor] = None, cross_head: bool = True,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """codes uint8 [slots, n_kv_heads, block_tokens, bits/8]; q_codes uint8 [n_req, n_q_heads, bits/8]."""
    _need_cuda(codes, req_offsets, q_codes, slot_ids, out)
    if codes.dtype != torch.uint8 or codes.dim() != 4 or not codes.is_contiguous():
        raise ValueError("codes must be contiguous uint8 [slots, n_kv_heads, block_tokens, bits/8]")
    if q_codes.dtype != torch.uint8 or q_codes.dim() != 3 or not q_codes.is_contiguous():
        raise ValueError("q_codes must be contiguous uint8 [n_req, n_q_heads, bits/8]")
    _, H, T, nb = codes.shape
    n_req = req_offsets.numel() - 1
    if q_codes.shape[0] != n_req or q_codes.shape[2] != nb:
        raise ValueError("q_codes shape does not match")
    if out is None:
        out = torch.empty((total,), dtype=torch.int32, device=codes.device)
    st = N.lib.ucmx_score_hamming(_ptr(codes), codes.shape[0], H, T, nb * 8, _ptr(_i32(req_offsets, "req_offsets")),
                                  _ptr(_i32(slot_ids, "slot_ids")), _ptr(q_codes), q_codes.shape[1], n_req, total,
                                  int(cross_head), _ptr(out), _stream(codes))
    N.check("ucmx_score_hamming", st, 1 if total and n_req else 0)
    return out


def topk_ragged(scores: torch.Tensor, req_offsets: torch.Tensor, k_per_req: torch.Tensor, *, out_stride: int,
                start_win: int = 0, end_win: int = 0, window_mode: int = WIN_NONE,
                order: int = ORDER_SCORE_DESC, id_map: Optional[torch.Tensor] = None, want_scores: bool = True,
                out_offsets: Optional[torch.Tensor] = None, out_idx: Optional[torch.Tensor] = None, out_scores: Optional[torch.Tensor] = None,
                out_counts: Optional[torch.Tensor] = None):
    """Per-request top-k. Returns (idx int32 [n_req, out_stride], scores or None, counts int32 [n_req]).
    Entries of a row beyond its count are -1 (indices) when this function allocates the output.
    With out_offsets (int32 [n_req+1]) the rows are packed back to back into flat outputs that the
    caller provides (out_idx, and out_scores if wanted, of out_offsets[-1] entries)."""
    _need_cuda(scores, req_offsets, k_per_req, id_map, out_idx, out_scores, out_counts)
    if scores.dtype == torch.float32:
        dt = DT_F32
    elif scores.dtype == torch.int32:
        dt = DT_I32
    else:
        raise ValueError("scores must be fp32 or int32")
    n_req = req_offsets.numel() - 1
    dev = scores.device
    if out_offsets is not None and out_idx is None:
        raise ValueError("packed output needs caller-provided out_idx")
    if out_idx is None:
        out_idx = torch.full((n_req, out_stride), -1, dtype=torch.int32, device=dev)
    if out_scores is None and want_scores and out_offsets is None:
        out_scores = torch.zeros((n_req, out_stride), dtype=scores.dtype, device=dev)
    if out_counts is None:
        out_counts = torch.zeros((n_req,), dtype=torch.int32, device=dev)
    st = N.lib.ucmx_topk_ragged(_ptr(scores), dt, _ptr(_i32(req_offsets, "req_offsets")),
                                _ptr(_i32(k_per_req, "k_per_req")), n_req, start_win, end_win, window_mode, order,
                                _ptr(_i32(id_map, "id_map")), out_stride, _ptr(_i32(out_offsets, "out_offsets")),
                                _ptr(out_idx), _ptr(out_scores),
                                _ptr(out_counts), _stream(scores))
    N.check("ucmx_topk_ragged", st, 1 if n_req else 0)
    return out_idx, out_scores, out_counts


def hash_encode(x: torch.Tensor, w: torch.Tensor, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x bf16 [..., dim], w bf16 [dim, bits] -> uint8 [..., bits/8] (LSB-first packed sign bits)."""
    _need_cuda(x, w, out)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or w.dim() != 2:
        raise ValueError("x and w must be bf16; w is [dim, bits]")
    dim, bits = w.shape
    if x.shape[-1] != dim:
        raise ValueError(f"x must be of shape (..., {dim}), but got {tuple(x.shape)}")
    x2 = x.reshape(-1, dim)
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    w = w.contiguous()
    if out is None:
        out = torch.empty(tuple(x.shape[:-1]) + (bits // 8,), dtype=torch.uint8, device=x.device)
    st = N.lib.ucmx_hash_encode(_ptr(x2), x2.shape[0], x2.stride(0), _ptr(w), dim, bits, _ptr(out), _stream(x))
    N.check("ucmx_hash_encode", st, 1 if x2.shape[0] else 0)
    return out


def hash_encode_blocks(k_cache: torch.Tensor, block_ids: torch.Tensor, w: torch.Tensor, *,
                       out_slots: Optional[torch.Tensor] = None, head_major: bool = True,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Hash codes of whole paged blocks -> uint8 [n, n_kv_heads, block_tokens, bits/8] (head_major) or
    [n, block_tokens, n_kv_heads, bits/8]."""
    _need_cuda(k_cache, block_ids, w, out_slots, out)
    g = kv_geometry(k_cache)
    ids = _i32(block_ids, "block_ids")
    dim, bits = w.shape
    if dim != g.head_dim or w.dtype != torch.bfloat16:
        raise ValueError("w must be bf16 [head_dim, bits]")
    n = ids.numel()
    if out is None:
        shape = (n, g.n_kv_heads, g.block_tokens, bits // 8) if head_major else (n, g.block_tokens, g.n_kv_heads, bits // 8)
        out = torch.empty(shape, dtype=torch.uint8, device=k_cache.device)
    rows = out.numel() // (g.n_kv_heads * g.block_tokens * (bits // 8))   # rows of the code table
    st = N.lib.ucmx_hash_encode_blocks(_ptr(k_cache), C.byref(g), _ptr(ids), _ptr(_i32(out_slots, "out_slots")), rows, n,
                                       _ptr(w.contiguous()), bits, int(head_major), _ptr(out), _stream(k_cache))
    N.check("ucmx_hash_encode_blocks", st, 1 if n else 0)
    return out


def _planes(planes: Sequence[torch.Tensor]):
    if not 1 <= len(planes) <= 8:
        raise ValueError("1..8 planes")
    arr = (C.c_void_p * len(planes))()
    for i, p in enumerate(planes):
        arr[i] = p.data_ptr()
    return arr


def _block_layout(planes: Sequence[torch.Tensor]):
    p0 = planes[0]
    esz = p0.element_size()
    stride_b = p0.stride(0) * esz
    inner = p0[0]
    if not inner.is_contiguous():
        raise ValueError("each block slice of a plane must be contiguous")
    slice_bytes = inner.numel() * esz
    for p in planes[1:]:
        if p.stride(0) * p.element_size() != stride_b or p[0].numel() * p.element_size() != slice_bytes:
            raise ValueError("planes must share block stride and slice size")
    return stride_b, slice_bytes


def gather_blocks(planes: Sequence[torch.Tensor], block_ids: torch.Tensor, staging: torch.Tensor) -> torch.Tensor:
    """Copy blocks block_ids[i] of every plane into staging laid out [i][plane][slice bytes].

    staging: a CUDA tensor, or a pinned CPU tensor (written directly over the host link)."""
    _need_cuda(block_ids, *planes)
    stride_b, slice_bytes = _block_layout(planes)
    ids = _i32(block_ids, "block_ids")
    n = ids.numel()
    host = not staging.is_cuda
    if host and not staging.is_pinned():
        raise ValueError("host staging must be pinned")
    if staging.numel() * staging.element_size() < n * len(planes) * slice_bytes:
        raise ValueError("staging too small")
    st = N.lib.ucmx_gather_blocks(_planes(planes), len(planes), stride_b, planes[0].shape[0], _ptr(ids), n, slice_bytes,
                                  _ptr(staging), int(host), _stream(planes[0]))
    N.check("ucmx_gather_blocks", st, 1 if n else 0)
    return staging


def scatter_blocks(planes: Sequence[torch.Tensor], block_ids: torch.Tensor, staging: torch.Tensor) -> None:
    """Inverse of gather_blocks: staging[i][plane] -> block block_ids[i] of each plane."""
    _need_cuda(block_ids, *planes)
    stride_b, slice_bytes = _block_layout(planes)
    ids = _i32(block_ids, "block_ids")
    n = ids.numel()
    host = not staging.is_cuda
    if host and not staging.is_pinned():
        raise ValueError("host staging must be pinned")
    if staging.numel() * staging.element_size() < n * len(planes) * slice_bytes:
        raise ValueError("staging too small")
    st = N.lib.ucmx_scatter_blocks(_planes(planes), len(planes), stride_b, planes[0].shape[0], _ptr(ids), n, slice_bytes,
                                   _ptr(staging), int(host), _stream(planes[0]))
    N.check("ucmx_scatter_blocks", st, 1 if n else 0)


def move_blocks(src_planes: Sequence[torch.Tensor], src_ids, dst_planes: Sequence[torch.Tensor],
                dst_ids: Optional[torch.Tensor] = None) -> None:
    """Block src_ids[i] of every source plane -> block dst_ids[i] of the matching destination plane (device memory on
    both sides); an entry with a negative id on either side is skipped.  This is the delta load of a decode step.
    src_ids may be a MoveList that remap_resident filled: its device-side length decides how many entries move, and
    the list is empty again afterwards."""
    moves = src_ids if isinstance(src_ids, MoveList) else None
    if moves is not None:
        src_ids, dst_ids = moves.src, moves.dst
    _need_cuda(src_ids, dst_ids, *src_planes, *dst_planes)
    if len(src_planes) != len(dst_planes):
        raise ValueError("as many destination planes as source planes")
    s_stride, slice_bytes = _block_layout(src_planes)
    d_stride, d_slice = _block_layout(dst_planes)
    if d_slice != slice_bytes:
        raise ValueError("source and destination blocks differ in size")
    sid, did = _i32(src_ids, "src_ids"), _i32(dst_ids, "dst_ids")
    if sid.numel() != did.numel():
        raise ValueError("one destination id per source id")
    n = sid.numel()
    st = N.lib.ucmx_move_blocks(_planes(src_planes), _planes(dst_planes), len(src_planes), s_stride, src_planes[0].shape[0],
                                _ptr(sid), d_stride, dst_planes[0].shape[0], _ptr(did), n,
                                None if moves is None else _ptr(moves.count), slice_bytes, _stream(src_planes[0]))
    N.check("ucmx_move_blocks", st, 1 if n else 0)


def copy_batch(dst_ptrs: torch.Tensor, src_ptrs: torch.Tensor, count: int, *, any_host_memory: bool = False) -> None:
    """dst_ptrs/src_ptrs: CUDA int64 tensors of addresses; copies `count` bytes per pair."""
    _need_cuda(dst_ptrs, src_ptrs)
    if dst_ptrs.dtype != torch.int64 or src_ptrs.dtype != torch.int64 or dst_ptrs.numel() != src_ptrs.numel():
        raise ValueError("pointer tensors must be int64 and of equal length")
    n = dst_ptrs.numel()
    st = N.lib.ucmx_copy_batch(_ptr(dst_ptrs), _ptr(src_ptrs), n, count, int(any_host_memory), _stream(dst_ptrs))
    N.check("ucmx_copy_batch", st, 1 if n and count else 0)


class MoveList:
    """One list of block moves for a whole batch, built on the device by remap_resident and consumed by move_blocks:
    src[i] -> dst[i] for i < count[0].  count is two int32 (the length and the mover's scratch), zero between rounds."""

    def __init__(self, capacity: int, device: torch.device):
        self.src = torch.full((capacity,), -1, dtype=torch.int32, device=device)
        self.dst = torch.full((capacity,), -1, dtype=torch.int32, device=device)
        self.count = torch.zeros((2,), dtype=torch.int32, device=device)
        self.capacity = capacity


def remap_resident(slot_logical: torch.Tensor, slot_free: torch.Tensor, slot_phys: torch.Tensor,
                   slot_offsets: torch.Tensor, sel: torch.Tensor, sel_offsets: torch.Tensor, *, max_logical: int,
                   max_slots: int, sel_counts: Optional[torch.Tensor] = None, src_map: Optional[torch.Tensor] = None,
                   src_map_offsets: Optional[torch.Tensor] = None, moves: Optional[MoveList] = None,
                   out: Optional[tuple] = None):
    """One round of the resident-set remap for every request (state tensors are updated in place).

    slot_logical int32, slot_free uint8, slot_phys int32: flat per-request state (CSR by slot_offsets);
    sel: ascending selected logical blocks (CSR by sel_offsets).  Returns (table, load_logical, load_phys,
    load_counts): table[j] = physical block serving sel[j]; the load lists are packed like sel, unused entries -1.
    With `moves` (and src_map, optionally src_map_offsets) the loads of all requests are also appended to that list
    as (src_map[src_map_offsets[r] + logical block] -> HBM block), ready for move_blocks.
    out: the result tensors of an earlier call, to be reused."""
    _need_cuda(slot_logical, slot_free, slot_phys, slot_offsets, sel, sel_offsets, sel_counts, src_map, src_map_offsets)
    if slot_free.dtype != torch.uint8 or not slot_free.is_contiguous():
        raise ValueError("slot_free must be contiguous uint8")
    n_req = slot_offsets.numel() - 1
    dev = sel.device
    if out is None:
        table = torch.full((sel.numel(),), -1, dtype=torch.int32, device=dev)
        load_logical = torch.full((sel.numel(),), -1, dtype=torch.int32, device=dev)
        load_phys = torch.full((sel.numel(),), -1, dtype=torch.int32, device=dev)
        load_counts = torch.zeros((n_req,), dtype=torch.int32, device=dev)
    else:
        table, load_logical, load_phys, load_counts = out[:4]
    mv = None
    if moves is not None:
        if src_map is None or moves.capacity < sel.numel():
            raise ValueError("a move list needs src_map and room for every selected block")
        mv = C.byref(N.RemapMoves(_i32(src_map, "src_map").data_ptr(),
                                  0 if src_map_offsets is None else _i32(src_map_offsets, "src_map_offsets").data_ptr(),
                                  moves.src.data_ptr(), moves.dst.data_ptr(), moves.count.data_ptr()))
    st = N.lib.ucmx_remap_resident(_ptr(_i32(slot_logical, "slot_logical")), _ptr(slot_free), _ptr(_i32(slot_phys, "slot_phys")),
                                   _ptr(_i32(slot_offsets, "slot_offsets")), _ptr(_i32(sel, "sel")),
                                   _ptr(_i32(sel_offsets, "sel_offsets")), _ptr(_i32(sel_counts, "sel_counts")), n_req,
                                   max_logical, max_slots, _ptr(table), _ptr(load_logical), _ptr(load_phys),
                                   _ptr(load_counts), mv, _stream(sel))
    N.check("ucmx_remap_resident", st, 1 if n_req else 0)
    return table, load_logical, load_phys, load_counts


def kvstar_block_repre(k_cache: torch.Tensor, block_ids: torch.Tensor, *, merge: int = 1,
                       pruned_index: Optional[torch.Tensor] = None, out_slots: Optional[torch.Tensor] = None,
                       out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """KVStar block representations: fp16 [slot, T/merge, H, d_pruned] from a bf16 paged cache.

    pruned_index: int64 [H, d_pruned] channels to keep per head (None keeps all)."""
    _need_cuda(k_cache, block_ids, pruned_index, out_slots, out)
    g = kv_geometry(k_cache)
    ids = _i32(block_ids, "block_ids")
    n = ids.numel()
    if pruned_index is not None:
        if pruned_index.dtype != torch.int64 or not pruned_index.is_contiguous() or pruned_index.shape[0] != g.n_kv_heads:
            raise ValueError("pruned_index must be contiguous int64 [n_kv_heads, d_pruned]")
        dp = pruned_index.shape[1]
    else:
        dp = g.head_dim
    if g.block_tokens % merge:
        raise ValueError("block_tokens must be a multiple of merge")
    M = g.block_tokens // merge
    if out is None:
        out = torch.empty((n, M, g.n_kv_heads, dp), dtype=torch.float16, device=k_cache.device)
    if out.dtype != torch.float16 or not out.is_contiguous() or tuple(out.shape[1:]) != (M, g.n_kv_heads, dp):
        raise ValueError("out must be contiguous fp16 [n_slots, T/merge, n_kv_heads, d_pruned]")
    st = N.lib.ucmx_kvstar_block_repre(_ptr(k_cache), C.byref(g), _ptr(ids), _ptr(_i32(out_slots, "out_slots")), out.shape[0], n,
                                       _ptr(pruned_index), dp, merge, _ptr(out), _stream(k_cache))
    N.check("ucmx_kvstar_block_repre", st, 1 if n else 0)
    return out


def kvstar_workspace_bytes(total: int, n_req: int, max_q_tokens: int, n_q_heads: int, n_kv_heads: int) -> int:
    return int(N.lib.ucmx_kvstar_workspace_bytes(total, n_req, max_q_tokens, n_q_heads, n_kv_heads))


def kvstar_scores(reps: torch.Tensor, req_offsets: torch.Tensor, q: torch.Tensor, q_offsets: torch.Tensor, *,
                  total: int, max_q_tokens: int, slot_ids: Optional[torch.Tensor] = None,
                  pruned_index: Optional[torch.Tensor] = None, workspace: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """KVStar softmax votes of every candidate block.

    reps fp16 [n_slots, M, H, d_pruned]; q fp16 [sum of query tokens, Hq, d_orig]; q_offsets int32 [n_req+1];
    req_offsets int32 [n_req+1] over slot_ids (or over table rows); pruned_index int64 [n_req, H, d_pruned]."""
    _need_cuda(reps, req_offsets, q, q_offsets, slot_ids, pruned_index, workspace, out)
    if reps.dim() != 4 or reps.dtype != torch.float16 or not reps.is_contiguous():
        raise ValueError("reps must be contiguous fp16 [n_slots, M, n_kv_heads, d_pruned]")
    if q.dim() != 3 or q.dtype != torch.float16 or not q.is_contiguous():
        raise ValueError("q must be contiguous fp16 [tokens, n_q_heads, head_dim]")
    n_slots, M, H, dp = reps.shape
    n_req = req_offsets.numel() - 1
    if q_offsets.numel() != n_req + 1:
        raise ValueError("q_offsets and req_offsets describe different numbers of requests")
    if pruned_index is not None and (pruned_index.dtype != torch.int64 or not pruned_index.is_contiguous()
                                     or tuple(pruned_index.shape) != (n_req, H, dp)):
        raise ValueError("pruned_index must be contiguous int64 [n_req, n_kv_heads, d_pruned]")
    need = kvstar_workspace_bytes(total, n_req, max_q_tokens, q.shape[1], H)
    if workspace is None:
        workspace = torch.empty((need,), dtype=torch.uint8, device=reps.device)
    if out is None:
        out = torch.empty((total,), dtype=torch.float32, device=reps.device)
    st = N.lib.ucmx_kvstar_scores(_ptr(reps), n_slots, M, H, dp, _ptr(_i32(req_offsets, "req_offsets")),
                                  _ptr(_i32(slot_ids, "slot_ids")), n_req, total, _ptr(q), _ptr(_i32(q_offsets, "q_offsets")),
                                  max_q_tokens, q.shape[1], q.shape[2], _ptr(pruned_index), _ptr(workspace),
                                  workspace.numel() * workspace.element_size(), _ptr(out), _stream(reps))
    N.check("ucmx_kvstar_scores", st, 3 if total and n_req else 0)
    return out
