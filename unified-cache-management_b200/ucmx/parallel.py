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
    """Partial block scores exchanged through peer-mapped memory and summed inside the top-k kernel
    (ucmx_peer_signal + ucmx_topk_ragged_peer_sum) instead of a library all-reduce between two kernels.

    Each rank owns one buffer every rank can address: 128 bytes of flags followed by two halves of
    `n_scores` fp32 partial scores that alternate from round to round.  `bases` lists the buffers'
    addresses in rank order; with torch.distributed they come from symmetric memory (`create`), and a
    test can pass plain allocations of one device to emulate several ranks in one process."""

    FLAG_BYTES = 128

    def __init__(self, bases: Sequence[int], my_rank: int, n_scores: int, device: torch.device, local: torch.Tensor):
        self.world, self.my_rank, self.n, self.device = len(bases), my_rank, n_scores, device
        self.local = local                                    # this rank's buffer as a float32 tensor
        self.bases_dev = torch.tensor(list(bases), dtype=torch.int64, device=device)
        self.half_bytes = ((n_scores * 4 + 127) // 128) * 128
        self.epoch = 0
        self.summed = torch.empty((n_scores,), dtype=torch.float32, device=device)

    @staticmethod
    def words_needed(n_scores: int) -> int:
        half = ((n_scores * 4 + 127) // 128) * 128
        return (PeerScoreExchange.FLAG_BYTES + 2 * half) // 4

    @classmethod
    def create(cls, n_scores: int, device: torch.device, group=None) -> "PeerScoreExchange":
        import torch.distributed._symmetric_memory as symm
        group = group if group is not None else dist.group.WORLD
        buf = symm.empty(cls.words_needed(n_scores), dtype=torch.float32, device=device)
        buf.zero_()
        hdl = symm.rendezvous(buf, group)
        torch.cuda.synchronize(device)
        dist.barrier(group=group)
        obj = cls([int(p) for p in hdl.buffer_ptrs], hdl.rank, n_scores, device, buf)
        obj._handle = hdl
        return obj

    def parts(self) -> torch.Tensor:
        """Where this round's partial scores go (a view into this rank's buffer); call begin_round first."""
        off = (self.FLAG_BYTES + (self.epoch & 1) * self.half_bytes) // 4
        return self.local[off: off + self.n]

    def begin_round(self) -> torch.Tensor:
        self.epoch += 1
        return self.parts()

    def signal(self) -> None:
        from . import _native as N
        import ctypes as C
        st = N.lib.ucmx_peer_signal(C.c_void_p(self.bases_dev.data_ptr()), self.world, self.my_rank, self.epoch,
                                    C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        N.check("ucmx_peer_signal", st, 1)

    def topk(self, req_offsets: torch.Tensor, k_per_req: torch.Tensor, *, out_stride: int, order: int, out_idx: torch.Tensor,
             out_counts: torch.Tensor, id_map: Optional[torch.Tensor] = None, out_offsets: Optional[torch.Tensor] = None,
             out_scores: Optional[torch.Tensor] = None, start_win: int = 0, end_win: int = 0, window_mode: int = 0) -> None:
        from . import _native as N
        import ctypes as C
        p = lambda t: C.c_void_p(0 if t is None else t.data_ptr())  # noqa: E731
        parts_off = self.FLAG_BYTES + (self.epoch & 1) * self.half_bytes
        st = N.lib.ucmx_topk_ragged_peer_sum(p(self.bases_dev), self.world, self.my_rank, parts_off, self.epoch, p(self.summed),
                                             p(req_offsets), p(k_per_req), req_offsets.numel() - 1, start_win, end_win,
                                             window_mode, order, p(id_map), out_stride, p(out_offsets), p(out_idx),
                                             p(out_scores), p(out_counts),
                                             C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream))
        N.check("ucmx_topk_ragged_peer_sum", st, 1)
