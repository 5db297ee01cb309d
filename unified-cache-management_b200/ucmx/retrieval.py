"""RetrievalWorkerBackend / RetrievalWorker with the interface of the reference's ESA native
back-end (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:17-225 and
ucm/sparse/esa/retrieval/retrieval_worker.py:10-34), backed by the device-resident object of the
C ABI (ucmx_retrieval_*): the representative table lives in HBM; submit() stores the request and
returns at once, and everything submitted since the last launch goes to the GPU as one ragged
score + top-k on a private stream when the first of those requests is polled, waited for or
collected (or on flush()).  poll() is an event query.

Host arrays in, host arrays out: submit copies the query and the index matrix to the device,
get_result returns numpy arrays, exactly like the pybind11 module it replaces.  Errors the
reference raises as std::runtime_error surface as RuntimeError with the same text.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _native as N


class RetrievalWorkerBackend:
    def __init__(self, data, *, device: int = 0, table_dtype: str = "bf16"):
        """data: float32 [n_items, dim] (numpy array or CPU torch tensor).

        table_dtype "bf16" keeps the table as bf16 in HBM, which loses nothing when the rows are
        bf16-rounded representatives (what ESA stores); "f32" keeps the reference's fp32 table."""
        arr = np.ascontiguousarray(_as_numpy(data), dtype=np.float32)
        if arr.ndim != 2:
            raise RuntimeError("data must be [n_items, dim]")
        self.n_items, self.dim = arr.shape
        self._h = C.c_void_p()
        dt = N.DT_BF16 if table_dtype == "bf16" else N.DT_F32
        st = N.lib.ucmx_retrieval_create(arr.ctypes.data_as(C.c_void_p), self.n_items, self.dim, dt, device,
                                         C.byref(self._h))
        N.check("ucmx_retrieval_create", st, 0)
        self._shapes = {}                      # request id -> (rows, k) of its result

    # -- the reference's four methods -------------------------------------------------------------
    def submit(self, query, topk: int, indexes) -> int:
        # arrays that are already what the C side reads (the common case) go through untouched
        q = query if _is_plain(query, np.float32) else np.ascontiguousarray(_as_numpy(query), dtype=np.float32)
        idx = indexes if _is_plain(indexes, np.int32) else np.ascontiguousarray(_as_numpy(indexes), dtype=np.int32)
        if q.ndim != 2 or q.shape[1] != self.dim:
            raise RuntimeError("Query dim mismatch")
        if idx.ndim != 2 or idx.shape[0] != q.shape[0]:
            raise RuntimeError("Query and indexes batch mismatch")
        rid = C.c_int32(-1)
        st = _submit(self._h, q.__array_interface__["data"][0], q.shape[0], q.shape[1], int(topk),
                     idx.__array_interface__["data"][0], idx.shape[1], C.byref(rid))
        if st != N.OK:
            N.check("ucmx_retrieval_submit", st, 0)
        self._shapes[rid.value] = (q.shape[0], min(int(topk), idx.shape[1]))
        return rid.value

    def flush(self) -> None:
        """Send everything submitted so far to the GPU now (otherwise the first poll/wait/get_result does it)."""
        N.check("ucmx_retrieval_flush", N.lib.ucmx_retrieval_flush(self._h), 0)

    def poll(self, req_id: int) -> bool:
        ready = C.c_int32(0)
        N.check("ucmx_retrieval_poll", N.lib.ucmx_retrieval_poll(self._h, req_id, C.byref(ready)), 0)
        return bool(ready.value)

    def wait(self, req_id: int) -> None:
        st = _wait(self._h, req_id)
        if st == N.ENOOBJ:
            raise RuntimeError("Bad req_id")
        if st != N.OK:
            N.check("ucmx_retrieval_wait", st, 0)

    def get_result(self, req_id: int) -> dict:
        shape = self._shapes.get(req_id)
        if shape is None:
            raise RuntimeError("Result not ready")
        indices = np.empty(shape, np.int32)
        scores = np.empty(shape, np.float32)
        st = _get(self._h, req_id, indices.__array_interface__["data"][0], scores.__array_interface__["data"][0])
        if st == N.ENOOBJ:
            raise RuntimeError("Result not ready")
        del self._shapes[req_id]
        if st != N.OK:
            N.check("ucmx_retrieval_get_result", st, 0)
        return {"indices": indices, "scores": scores}

    # -- additions ---------------------------------------------------------------------------------
    def update_rows(self, slots, rows) -> None:
        """data[slots] = rows, ordered before later submits (the reference mutates its numpy table
        in place under the worker threads, ucm/sparse/esa/esa.py:364)."""
        s = np.ascontiguousarray(_as_numpy(slots), dtype=np.int32)
        r = np.ascontiguousarray(_as_numpy(rows), dtype=np.float32).reshape(len(s), self.dim)
        st = N.lib.ucmx_retrieval_update_rows(self._h, s.ctypes.data_as(C.c_void_p), len(s),
                                              r.ctypes.data_as(C.c_void_p))
        N.check("ucmx_retrieval_update_rows", st, 1)

    @property
    def launches(self) -> int:
        """Kernels this object has launched so far (one ragged score + one top-k per batch of submits)."""
        n = C.c_int64(0)
        N.check("ucmx_retrieval_launches", N.lib.ucmx_retrieval_launches(self._h, C.byref(n)), 0)
        return n.value

    def table_ptr(self):
        p, dt = C.c_void_p(), C.c_int32(0)
        N.check("ucmx_retrieval_table", N.lib.ucmx_retrieval_table(self._h, C.byref(p), C.byref(dt)), 0)
        return p.value, dt.value

    def close(self) -> None:
        if self._h:
            N.lib.ucmx_retrieval_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


_submit = N.lib.ucmx_retrieval_submit
_wait = N.lib.ucmx_retrieval_wait
_get = N.lib.ucmx_retrieval_get_result


def _is_plain(x, dtype) -> bool:
    return type(x) is np.ndarray and x.dtype == dtype and x.flags.c_contiguous


def _as_numpy(x):
    if isinstance(x, np.ndarray):
        return x
    if hasattr(x, "detach"):          # torch tensor
        x = x.detach()
        if x.is_cuda:
            x = x.to("cpu")
        if str(x.dtype) == "torch.bfloat16":
            x = x.float()
        return x.numpy()
    return np.asarray(x)


class RetrievalWorker:
    """torch -> numpy and float16/bfloat16 -> float32 conversion in front of the back-end
    (ucm/sparse/esa/retrieval/retrieval_worker.py:10-34)."""

    def __init__(self, cpp_worker: RetrievalWorkerBackend):
        self.cpp_worker = cpp_worker

    @classmethod
    def handle_input(cls, input):
        return np.ascontiguousarray(_as_numpy(input), dtype=np.float32)

    def submit(self, query, topk, indexes):
        return self.cpp_worker.submit(self.handle_input(query), topk, indexes)

    def poll(self, req_id):
        return self.cpp_worker.poll(req_id)

    def get_result(self, req_id):
        return self.cpp_worker.get_result(req_id)

    def wait(self, req_id):
        return self.cpp_worker.wait(req_id)
