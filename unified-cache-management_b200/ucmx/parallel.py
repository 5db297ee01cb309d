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
