"""Multi-GPU sharding of the retrieval path (one process per GPU, torch.distributed for plumbing).

Two independent ways to shard, both of which the path offers naturally:
  * data parallel over requests - every request's pool/score/top-k/gather is independent, so the
    ragged batch is split by block count and no data crosses GPUs;
  * tensor parallel over KV heads - the way the serving engine already shards the KV cache.  A block's
    score is a sum over heads, so each rank scores its own heads and one all-reduce (sum) of the
    per-block scores precedes top-k, which every rank then computes identically.  The reference
    has no such exchange: under tensor parallelism its ranks select independently over their own
    heads (ucm/sparse/esa/esa.py:196-198) and may disagree.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist


def partition_requests(blocks_per_req: Sequence[int], world_size: int) -> List[List[int]]:
    """Split request indices over ranks so that block counts are balanced (largest first, to the
    least loaded rank).  Deterministic; every rank computes the same answer."""
    order = sorted(range(len(blocks_per_req)), key=lambda i: (-int(blocks_per_req[i]), i))
    loads = [0] * world_size
    parts: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        parts[r].append(i)
        loads[r] += int(blocks_per_req[i])
    return [sorted(p) for p in parts]


def head_range(n_kv_heads: int, rank: int, world_size: int) -> Tuple[int, int]:
    """KV heads [lo, hi) held by `rank` (contiguous, equal shares; world_size must divide n_kv_heads)."""
    if n_kv_heads % world_size:
        raise ValueError("tensor-parallel size must divide the number of KV heads")
    per = n_kv_heads // world_size
    return rank * per, (rank + 1) * per


class ScoreAllReduce:
    """In-place sum of per-block scores over the tensor-parallel group (fp32 for dot scores, int32
    for Hamming scores - integer sums stay exact).  NCCL on CUDA tensors, gloo on CPU tensors."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None):
        self.group = group
        self.calls = 0

    def __call__(self, scores: torch.Tensor) -> torch.Tensor:
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(scores, op=dist.ReduceOp.SUM, group=self.group)
        self.calls += 1
        return scores


def max_over_ranks(value: float, device: torch.device) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class PeerScoreExchange:
    """The all-reduce of partial block scores, carried by the scoring and top-k kernels themselves over peer
    memory instead of a library collective between them (ucmx_score_dot* with an exchange + ucmx_topk_ragged_peer_sum).

    Each rank owns one buffer every rank can address: a 256-byte header (one flag per rank, this rank's arrival and
    round counters) followed by an inbox of two halves x world parts of `n_scores` fp32 partial scores.  A rank's
    scoring kernel stores its scores into its part of EVERY rank's inbox and, when its last thread block is done,
    publishes the round into its flag on every rank; the top-k kernel that follows waits (bounded) for all flags of
    its own buffer and adds the parts in rank order.  The round counter lives in the buffer and advances on the
    device, so score + top-k can be captured into a CUDA graph and replayed.  `bases` lists the buffers' addresses
    in rank order; with torch.distributed they come from symmetric memory (`create`), and a test can pass plain
    allocations of one device to emulate several ranks in one process (their launches then run one after the
    other: all scoring launches of a round first, then the top-k launches)."""

    def __init__(self, bases: Sequence[int], my_rank: int, n_scores: int, device: torch.device, local: torch.Tensor):
        from . import _native as N
        import ctypes as C
        self.world, self.my_rank, self.n, self.device = len(bases), my_rank, n_scores, device
        self.local = local                                    # this rank's buffer (keeps it alive)
        self.bases_dev = torch.tensor(list(bases), dtype=torch.int64, device=device)
        self.desc = N.PeerExchange(C.c_void_p(self.bases_dev.data_ptr()), self.world, my_rank, n_scores)
        self.summed = torch.empty((n_scores,), dtype=torch.float32, device=device)

    @staticmethod
    def words_needed(world: int, n_scores: int) -> int:
        from . import _native as N
        return (int(N.lib.ucmx_peer_exchange_bytes(world, n_scores)) + 3) // 4

    @classmethod
    def create(cls, n_scores: int, device: torch.device, group=None) -> "PeerScoreExchange":
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        world = dist.get_world_size(group)
        buf = symm.empty(cls.words_needed(world, n_scores), dtype=torch.float32, device=device)
        buf.zero_()
        hdl = symm.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        obj = cls([int(p) for p in hdl.buffer_ptrs], hdl.rank, n_scores, device, buf)
        obj._handle = hdl
        return obj

    def topk(self, req_offsets: torch.Tensor, k_per_req: torch.Tensor, *, total: int, out_stride: int, order: int,
             out_idx: torch.Tensor, out_counts: torch.Tensor, id_map: Optional[torch.Tensor] = None,
             out_offsets: Optional[torch.Tensor] = None, out_scores: Optional[torch.Tensor] = None, start_win: int = 0,
             end_win: int = 0, window_mode: int = 0) -> None:
        from . import _native as N
        import ctypes as C
        p = lambda t: C.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731
        st = N.lib.ucmx_topk_ragged_peer_sum(C.byref(self.desc), p(self.summed), p(req_offsets), p(k_per_req),
                                             req_offsets.numel() - 1, total, start_win, end_win, window_mode, order,
                                             p(id_map), out_stride, p(out_offsets), p(out_idx), p(out_scores),
                                             p(out_counts), C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        N.check("ucmx_topk_ragged_peer_sum", st, 1)
