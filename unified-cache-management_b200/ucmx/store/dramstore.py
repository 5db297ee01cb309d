"""Host-memory KV store on top of the batched transfer kernels.

Interface and behaviour follow the reference's UcmDramStore
(ucm/store/dramstore/dramstore_connector.py:54-227): keys are "<block id>_<offset>", dump() refuses
new data once the cache is full (the task then fails in wait()), load() of a key that was never
dumped raises KeyError.  What differs is the data path.  The reference issues one memcpy per block
slice from a Python loop and keeps one pageable CPU tensor per key; here the store owns one
page-locked slab (the IBufferedDevice idea, ucm/store/device/ibuffered_device.h:32-62) cut into
slots of `io_size` bytes, and a whole dump or load is ONE kernel launch over a device-resident
table of (source, destination) addresses (the H2DBatch/D2HBatch idea of
ucm/store/device/cuda/cuda_device.cu:47-81) on the store's own stream, ordered after the caller's
stream with an event instead of a host synchronisation.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

import numpy as np
import torch

from .. import _native as N
from .ucmstore import Task, UcmKVStoreBase

SUCCESS = 0
FAILURE = -1


@dataclass
class DramTask(Task):
    task_id: str = "1"
    handle: Optional[int] = None                 # ucmx_task*
    keep: List[Any] = field(default_factory=list)  # tensors the kernel still reads

    def __del__(self):  # pragma: no cover
        if self.handle:
            N.lib.ucmx_task_destroy(C.c_void_p(self.handle))
            self.handle = None


def store_offset(block_shape: Tuple[int, int, int], rank: int, tp_size: int, precision: int, layer_id: int,
                 is_v: bool, is_mla: bool = False) -> int:
    """Byte offset of one rank's K (or V) slice of one layer inside a stored block
    (get_offset, ucm/sparse/esa/esa.py:123-135)."""
    block_size, heads_per_tp, head_size = block_shape
    k_sz = block_size * heads_per_tp * head_size * precision
    v_sz = 0 if is_mla else k_sz
    layer_sz = (k_sz + v_sz) * tp_size
    k_off = layer_sz * layer_id if is_mla else layer_sz * layer_id + layer_sz // tp_size * rank
    return k_off + k_sz if is_v else k_off


class UcmDramStore(UcmKVStoreBase):
    def __init__(self, config: Dict):
        super().__init__(config)
        self.max_cache_byte = int(config.get("max_cache_size", 5368709120))
        self.kv_block_size = int(config.get("kv_block_size", 262144))
        self.io_size = int(config.get("io_size", self.kv_block_size))
        self.max_block_num = self.max_cache_byte // self.kv_block_size
        self.role = config.get("role", "worker")
        self.device = torch.device(config.get("device", "cuda:0")) if self.role != "scheduler" else None
        self.timeout_ms = int(config.get("transferTimeoutMs", 30000))
        self.cached_blocks = set()
        self.slot_of: Dict[str, int] = {}
        self._ring = None
        self._base = 0
        self._n_slots = 0
        self._stream: Optional[torch.cuda.Stream] = None
        self._staging: Optional[torch.Tensor] = None
        self.staging_bytes = int(config.get("staging_bytes", 1 << 30))

    # ------------------------------------------------------------------ slab
    def _ensure_slab(self) -> None:
        if self._ring is not None:
            return
        n_slots = max(1, self.max_cache_byte // self.io_size)
        ring = C.c_void_p()
        N.check("ucmx_ring_create", N.lib.ucmx_ring_create(self.io_size, n_slots, C.byref(ring)), 0)
        base, sb, ns = C.c_void_p(), C.c_size_t(), C.c_size_t()
        N.check("ucmx_ring_base", N.lib.ucmx_ring_base(ring, C.byref(base), C.byref(sb), C.byref(ns)), 0)
        self._ring, self._base, self._n_slots = ring, base.value, ns.value
        self._stream = torch.cuda.Stream(device=self.device)

    def _acquire(self) -> int:
        ptr, idx = C.c_void_p(), C.c_int32(-1)
        st = N.lib.ucmx_ring_acquire(self._ring, C.byref(ptr), C.byref(idx))
        return idx.value if st == N.OK else -1

    def slab_view(self, slot: int) -> np.ndarray:
        """The bytes of one slot (host memory), for inspection and tests."""
        buf = (C.c_uint8 * self.io_size).from_address(self._base + slot * self.io_size)
        return np.frombuffer(buf, dtype=np.uint8)

    # ------------------------------------------------------------------ interface
    def cc_store(self) -> int:
        return 0

    def create(self, block_ids: List[str]) -> List[int]:
        return [SUCCESS] * len(block_ids)

    def lookup(self, block_ids: List[str]) -> List[bool]:
        return [b in self.cached_blocks for b in block_ids]

    def prefetch(self, block_ids: List[str]) -> None:
        return None

    def _launch(self, dst: np.ndarray, src: np.ndarray, nbytes: int, keep: List[Any], to_host: bool) -> DramTask:
        """One batch of equal-sized copies dst[i] <- src[i] on the store's stream.

        When the host side of the batch is one contiguous run of slab slots (the usual case: slots
        are handed out in order) the batch goes in two steps - compaction through a device staging
        area plus ONE DMA over the host link - which measured faster than letting the kernel write
        host memory directly; otherwise the kernel copies each pair itself."""
        task = DramTask()
        n = len(dst)
        cur = torch.cuda.current_stream(self.device)
        self._stream.wait_stream(cur)
        sp = C.c_void_p(self._stream.cuda_stream)
        with torch.cuda.stream(self._stream):
            host = dst if to_host else src
            run = n > 1 and nbytes == self.io_size and bool(np.all(np.diff(host) == self.io_size))
            keep = list(keep)
            if run and n * nbytes <= self.staging_bytes:
                if self._staging is None or self._staging.numel() < n * nbytes:
                    self._staging = torch.empty(max(n * nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
                base = self._staging.data_ptr()
                stage_addr = base + np.arange(n, dtype=np.int64) * nbytes
                if to_host:
                    pairs = torch.from_numpy(np.stack([stage_addr, src])).to(self.device)
                    st = N.lib.ucmx_copy_batch(C.c_void_p(pairs[0].data_ptr()), C.c_void_p(pairs[1].data_ptr()), n, nbytes, 0, sp)
                    N.check("ucmx_copy_batch", st, 1)
                    N.check("ucmx_memcpy_async", N.lib.ucmx_memcpy_async(C.c_void_p(int(host[0])), C.c_void_p(base), n * nbytes, sp), 0)
                else:
                    N.check("ucmx_memcpy_async", N.lib.ucmx_memcpy_async(C.c_void_p(base), C.c_void_p(int(host[0])), n * nbytes, sp), 0)
                    pairs = torch.from_numpy(np.stack([dst, stage_addr])).to(self.device)
                    st = N.lib.ucmx_copy_batch(C.c_void_p(pairs[0].data_ptr()), C.c_void_p(pairs[1].data_ptr()), n, nbytes, 0, sp)
                    N.check("ucmx_copy_batch", st, 1)
                keep.append(self._staging)
            else:
                pairs = torch.from_numpy(np.stack([dst, src])).to(self.device)
                st = N.lib.ucmx_copy_batch(C.c_void_p(pairs[0].data_ptr()), C.c_void_p(pairs[1].data_ptr()), n, nbytes, 1, sp)
                N.check("ucmx_copy_batch", st, 1 if n else 0)
            h = C.c_void_p()
            N.check("ucmx_task_create", N.lib.ucmx_task_create(C.byref(h)), 0)
            N.check("ucmx_task_record", N.lib.ucmx_task_record(h, sp), 0)
        task.handle = h.value
        task.keep = keep + [pairs]
        return task

    def _addresses(self, tensors: List[torch.Tensor]) -> Tuple[np.ndarray, int]:
        if not tensors:
            return np.zeros(0, np.int64), 0
        nbytes = tensors[0].numel() * tensors[0].element_size()
        for t in tensors:
            if not t.is_cuda or not t.is_contiguous() or t.numel() * t.element_size() != nbytes:
                raise ValueError("transfer tensors must be contiguous CUDA tensors of one size")
        if nbytes > self.io_size or nbytes % 16:
            raise ValueError(f"slice of {nbytes} bytes does not fit io_size {self.io_size} (or is not a multiple of 16)")
        return np.fromiter((t.data_ptr() for t in tensors), dtype=np.int64, count=len(tensors)), nbytes

    def dump(self, block_ids: List[str], offset: List[int], src_tensor: List[torch.Tensor]) -> Task:
        self._ensure_slab()
        src, nbytes = self._addresses(src_tensor)
        if len(self.slot_of) + len(block_ids) > self.max_block_num * max(1, self.kv_block_size // self.io_size):
            return DramTask(task_id="-1")
        slots = []
        for i, b in enumerate(block_ids):
            key = f"{b}_{offset[i]}"
            s = self.slot_of.get(key)
            if s is None:
                s = self._acquire()
                if s < 0:
                    for k2, s2 in slots:       # roll back what this call took
                        if k2 is not None:
                            N.lib.ucmx_ring_release(self._ring, s2)
                            del self.slot_of[k2]
                    return DramTask(task_id="-1")
                self.slot_of[key] = s
                slots.append((key, s))
            else:
                slots.append((None, s))
        dst = np.asarray([self._base + s * self.io_size for _, s in slots], dtype=np.int64)
        return self._launch(dst, src, nbytes, list(src_tensor), True)

    def load(self, block_ids: List[str], offset: List[int], dst_tensor: List[torch.Tensor]) -> Task:
        self._ensure_slab()
        dst, nbytes = self._addresses(dst_tensor)
        src = np.asarray([self._base + self.slot_of[f"{b}_{offset[i]}"] * self.io_size for i, b in enumerate(block_ids)],
                         dtype=np.int64)
        return self._launch(dst, src, nbytes, list(dst_tensor), False)

    def fetch_data(self, block_ids: List[str], offset: List[int], dst_addr: List[int], size: List[int]) -> Task:
        self._ensure_slab()
        if len(set(size)) > 1:
            raise ValueError("one transfer moves slices of one size")
        src = np.asarray([self._base + self.slot_of[f"{b}_{offset[i]}"] * self.io_size for i, b in enumerate(block_ids)],
                         dtype=np.int64)
        return self._launch(np.asarray(dst_addr, dtype=np.int64), src, size[0] if size else 0, [], False)

    def dump_data(self, block_ids: List[str], offset: List[int], src_addr: List[int], size: List[int]) -> Task:
        self._ensure_slab()
        if len(set(size)) > 1:
            raise ValueError("one transfer moves slices of one size")
        slots, taken = [], []
        for i, b in enumerate(block_ids):
            key = f"{b}_{offset[i]}"
            s = self.slot_of.get(key)
            if s is None:
                s = self._acquire()
                if s < 0:
                    for k2, s2 in taken:       # roll back what this call took
                        N.lib.ucmx_ring_release(self._ring, s2)
                        del self.slot_of[k2]
                    return DramTask(task_id="-1")
                self.slot_of[key] = s
                taken.append((key, s))
            slots.append(s)
        dst = np.asarray([self._base + s * self.io_size for s in slots], dtype=np.int64)
        return self._launch(dst, np.asarray(src_addr, dtype=np.int64), size[0] if size else 0, [], True)

    def wait(self, task: DramTask) -> int:
        if task.task_id == "-1":
            return FAILURE
        if task.handle is None:
            return FAILURE
        st = N.lib.ucmx_task_wait(C.c_void_p(task.handle), self.timeout_ms)
        if st == N.OK:
            task.keep = []                     # the kernel is done with the tensors, tables and staging it borrowed
            return SUCCESS
        # Timed out or failed: the copy may still be running, so what it reads and writes stays referenced.  The
        # references go when a later check() or wait() sees the task finished, or with the task object itself.
        self._lingering = [t for t in getattr(self, "_lingering", []) if not self._finished(t)]
        self._lingering.append(task)
        return FAILURE

    def _finished(self, task: DramTask) -> bool:
        fin = C.c_int32(0)
        st = N.lib.ucmx_task_check(C.c_void_p(task.handle), C.byref(fin))
        if st == N.OK and fin.value:
            task.keep = []
            return True
        return False

    def commit(self, block_ids: List[str], is_success: bool = True) -> None:
        if is_success:
            self.cached_blocks.update(block_ids)

    def check(self, task: DramTask) -> Tuple[int, bool]:
        if task.task_id == "-1" or task.handle is None:
            return FAILURE, True
        fin = C.c_int32(0)
        st = N.lib.ucmx_task_check(C.c_void_p(task.handle), C.byref(fin))
        return (SUCCESS if st == N.OK else FAILURE), bool(fin.value)

    def close(self) -> None:
        if self._ring is not None:
            torch.cuda.synchronize(self.device)
            N.lib.ucmx_ring_destroy(self._ring)
            self._ring = None
