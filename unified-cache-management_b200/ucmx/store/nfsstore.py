"""File-per-block KV store (shared file system / local disk) on the native data plane.

Interface, configuration keys and on-disk format follow the reference's UcmNfsStore
(ucm/store/nfsstore/nfsstore_connector.py:39-125): `storage_backends` is a ':'-separated list of
directories, `kv_block_size` the fixed file size of a block, `role` == "worker" enables transfers,
`device` and `io_size` configure them.  Files written by either implementation can be read by the
other.  Disk I/O and the PCIe leg run in libucmx's worker threads (csrc/fstore.cu): groups of slices
are read into page-locked slots and cross to HBM in one kernel launch per group.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import torch

from .. import _native as N
from .ucmstore import Task, UcmKVStoreBase

DUMP, LOAD = 0, 1
HOST, DEVICE = 0, 1


@dataclass
class NfsTask(Task):
    task_id: int = 0


def _id_bytes(block_id) -> bytes:
    b = block_id if isinstance(block_id, (bytes, bytearray)) else str(block_id).encode()
    if len(b) < 16:
        raise ValueError("block ids must be at least 16 bytes long: the first 16 name the block's file")
    return bytes(b)


class UcmNfsStore(UcmKVStoreBase):
    def __init__(self, config: Dict):
        super().__init__(config)
        backends = ":".join(p for p in str(config["storage_backends"]).split(":") if p)
        block_size = int(config["kv_block_size"])
        transfer = config.get("role", "worker") == "worker"
        device = int(config.get("device", -1)) if transfer else -1
        handle = C.c_void_p()
        st = N.lib.ucmx_fstore_create(
            backends.encode(), block_size, 1 if config.get("temp_dump_dir_enable", False) else 0,
            1 if transfer else 0, device, int(config.get("io_size", 262144)),
            int(config.get("buffer_number", 0)), int(config.get("stream_number", 0)),
            int(config.get("timeout_ms", 0)), C.byref(handle))
        if st != N.OK:
            raise RuntimeError(f"Failed to initialize ucmnfsstore, errcode: {st}.")
        self._h = handle
        self.device = device

    def __del__(self):  # pragma: no cover
        h, self._h = getattr(self, "_h", None), None
        if h:
            N.lib.ucmx_fstore_destroy(h)

    def close(self) -> None:
        h, self._h = self._h, None
        if h:
            N.lib.ucmx_fstore_destroy(h)

    # ------------------------------------------------------------------ block files
    def cc_store(self) -> int:
        return int(self._h.value or 0)

    def create(self, block_ids: List[str]) -> List[int]:
        out = []
        for b in block_ids:
            raw = _id_bytes(b)
            out.append(int(N.lib.ucmx_fstore_alloc(self._h, raw, len(raw))))
        return out

    def lookup(self, block_ids: List[str]) -> List[bool]:
        out, found = [], C.c_int32(0)
        for b in block_ids:
            raw = _id_bytes(b)
            st = N.lib.ucmx_fstore_lookup(self._h, raw, len(raw), C.byref(found))
            out.append(st == N.OK and found.value != 0)
        return out

    def prefetch(self, block_ids: List[str]) -> None:
        pass

    def commit(self, block_ids: List[str], is_success: bool = True) -> None:
        for b in block_ids:
            raw = _id_bytes(b)
            N.lib.ucmx_fstore_commit(self._h, raw, len(raw), 1 if is_success else 0)

    def path(self, block_id, activated: bool = False) -> str:
        raw = _id_bytes(block_id)
        buf = C.create_string_buffer(4096)
        st = N.lib.ucmx_fstore_path(self._h, raw, len(raw), 1 if activated else 0, buf, 4096)
        if st != N.OK:
            raise N.UcmxError("ucmx_fstore_path", st)
        return buf.value.decode()

    # --------------------------------------------------------------------- transfers
    def _submit(self, kind: int, location: int, block_ids: Sequence, offsets: Sequence[int], addrs: Sequence[int],
                sizes: Sequence[int]) -> NfsTask:
        n = min(len(block_ids), len(offsets), len(addrs), len(sizes))   # the reference stops at the shortest list
        raws = [_id_bytes(b) for b in block_ids[:n]]
        ids = (C.c_char_p * n)(*raws)
        lens = (C.c_size_t * n)(*[len(r) for r in raws])
        offs = (C.c_size_t * n)(*[int(o) for o in offsets[:n]])
        adr = (C.c_size_t * n)(*[int(a) for a in addrs[:n]])
        szs = (C.c_size_t * n)(*[int(s) for s in sizes[:n]])
        tid = C.c_size_t(0)
        st = N.lib.ucmx_fstore_submit(self._h, kind, location, ids, lens, offs, adr, szs, n, C.byref(tid))
        # like the reference, a refused submit yields the invalid task id 0, which wait() reports
        return NfsTask(task_id=tid.value if st == N.OK else 0)

    @staticmethod
    def _location(tensors: List[torch.Tensor]) -> int:
        return DEVICE if tensors and tensors[0].is_cuda else HOST

    def load(self, block_ids: List[str], offset: List[int], dst_tensor: List[torch.Tensor]) -> Task:
        return self._submit(LOAD, self._location(dst_tensor), block_ids, offset, [t.data_ptr() for t in dst_tensor],
                            [t.numel() * t.element_size() for t in dst_tensor])

    def dump(self, block_ids: List[str], offset: List[int], src_tensor: List[torch.Tensor]) -> Task:
        loc = self._location(src_tensor)
        if loc == DEVICE:
            # the workers read the tensors on their own streams: what the caller queued must have landed
            torch.cuda.current_stream(src_tensor[0].device).synchronize()
        return self._submit(DUMP, loc, block_ids, offset, [t.data_ptr() for t in src_tensor],
                            [t.numel() * t.element_size() for t in src_tensor])

    def fetch_data(self, block_ids: List[str], offset: List[int], dst_addr: List[int], size: List[int]) -> Task:
        return self._submit(LOAD, DEVICE if self.device >= 0 else HOST, block_ids, offset, dst_addr, size)

    def dump_data(self, block_ids: List[str], offset: List[int], src_addr: List[int], size: List[int]) -> Task:
        return self._submit(DUMP, DEVICE if self.device >= 0 else HOST, block_ids, offset, src_addr, size)

    def load_to_host(self, block_ids, offset, dst_addr, size) -> Task:
        return self._submit(LOAD, HOST, block_ids, offset, dst_addr, size)

    def dump_from_host(self, block_ids, offset, src_addr, size) -> Task:
        return self._submit(DUMP, HOST, block_ids, offset, src_addr, size)

    def wait(self, task: Task) -> int:
        return int(N.lib.ucmx_fstore_wait(self._h, task.task_id))

    def check(self, task: Task) -> Tuple[int, bool]:
        fin = C.c_int32(0)
        st = N.lib.ucmx_fstore_check(self._h, task.task_id, C.byref(fin))
        return int(st), fin.value != 0
