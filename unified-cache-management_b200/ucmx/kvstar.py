"""Drop-in for the reference's `kvstar_retrieve` extension module (ucm/sparse/kvstar/retrieve/py_intf/py_intf.cpp:
Setup, AsyncRetrieveByCPU, Wait, GetTaskResult, DeviceType) on the GPU kernels.

The reference copies the query group and the block representations to the host and runs
KVStar::Execute on a CPU thread pool (ucm/sparse/kvstar/multistep.py:240-262).  Here the same call
enqueues the tensor-core scoring kernels and the top-k on a CUDA stream and returns at once; `Wait`
synchronises with the recorded event.  Tensors already on the device are used in place; host tensors
(what the reference passes) are copied over first.
"""
from __future__ import annotations

import enum
import itertools
import threading
from typing import Dict, Optional

import torch

from . import ops


class DeviceType(enum.IntEnum):
    CPU = 0
    NPU = 1
    GPU = 2


CPU = DeviceType.CPU
GPU = DeviceType.GPU

_tasks: Dict[int, dict] = {}
_ids = itertools.count(1)
_lock = threading.Lock()
_device: Optional[torch.device] = None


def Setup(param=None) -> int:
    """The reference sizes its CPU thread pool and NUMA allocator here; nothing of that is needed."""
    return 0


def _dev() -> torch.device:
    global _device
    if _device is None:
        if not torch.cuda.is_available():
            raise RuntimeError("ucmx.kvstar needs a CUDA device; there is no CPU path")
        _device = torch.device("cuda", torch.cuda.current_device())
    return _device


def AsyncRetrieveByCPU(query_group: torch.Tensor, blk_repre: torch.Tensor, d_pruned_index: Optional[torch.Tensor],
                       topk: int, req_id: int = 0, device=CPU) -> int:
    """query_group: half [x, Hq, d]; blk_repre: half [n, M, h, d_pruned]; d_pruned_index: int64 [h, d_pruned] or None.
    Returns a task id; the task's result is the indices (rows of blk_repre) of the topk highest-voted blocks."""
    if query_group.dim() != 3:
        raise RuntimeError("Query shape must be 3D (x, H, d).")
    if blk_repre.dim() != 4:
        raise RuntimeError("BlockRep shape must be 4D (n, M, h, d).")
    x, Hq, d = query_group.shape
    n, M, h, dp = blk_repre.shape
    if Hq % h:
        raise RuntimeError("Num_q_heads must be a divisible by num_kv_heads.")
    if d_pruned_index is not None and tuple(d_pruned_index.shape) != (h, dp):
        raise RuntimeError("dPrunedIndex shape is inconsistent with K's shape.")
    if d_pruned_index is None and d != dp:
        raise RuntimeError("Dimension mismatch: No dPrunedIndex, but Q and K head dims differ.")
    dev = _dev()
    q = query_group.to(device=dev, dtype=torch.float16, non_blocking=True).contiguous()
    reps = blk_repre.to(device=dev, dtype=torch.float16, non_blocking=True).contiguous()
    pr = None if d_pruned_index is None else d_pruned_index.to(device=dev, dtype=torch.int64).contiguous().unsqueeze(0)
    off = torch.tensor([0, n], dtype=torch.int32, device=dev)
    qoff = torch.tensor([0, x], dtype=torch.int32, device=dev)
    k = max(min(int(topk), n), 0)
    task = {"n": n, "k": k, "keep": (q, reps, pr, off, qoff)}
    if k > 0:
        votes = ops.kvstar_scores(reps, off, q, qoff, total=n, max_q_tokens=x, pruned_index=pr)
        kk = torch.tensor([k], dtype=torch.int32, device=dev)
        idx, _, _ = ops.topk_ragged(votes, off, kk, out_stride=k, order=ops.ORDER_SCORE_DESC)
        task["idx"] = idx
    ev = torch.cuda.Event()
    ev.record(torch.cuda.current_stream(dev))
    task["event"] = ev
    with _lock:
        tid = next(_ids)
        _tasks[tid] = task
    return tid


def Wait(task_id: int) -> int:
    with _lock:
        task = _tasks.get(task_id)
    if task is None:
        return -1
    task["event"].synchronize()
    return 0


def GetTaskResult(task_id: int):
    with _lock:
        task = _tasks.get(task_id)
    if task is None:
        return None
    if not task["event"].query():
        return {"status": "RUNNING"}
    data = [] if task["k"] == 0 else task["idx"].reshape(-1)[:task["k"]].to(torch.int64).cpu().tolist()
    task["keep"] = None
    return {"status": "SUCCESS", "data": data}


def ReleaseTask(task_id: int) -> None:
    with _lock:
        _tasks.pop(task_id, None)


def extract_block_repre(k_cache: torch.Tensor, vllm_block_ids, d_pruned_index: Optional[torch.Tensor], merge: int):
    """Block representations of the listed blocks (extract_block_repre, ucm/sparse/kvstar/multistep.py:279-316,
    followed by the half cast of :495-499), computed on the device."""
    ids = torch.as_tensor(vllm_block_ids, dtype=torch.int32, device=k_cache.device)
    pr = None if d_pruned_index is None else d_pruned_index.to(device=k_cache.device, dtype=torch.int64).contiguous()
    return ops.kvstar_block_repre(k_cache, ids, merge=merge, pruned_index=pr)
