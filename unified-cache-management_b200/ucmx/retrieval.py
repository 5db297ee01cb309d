"""RetrievalWorkerBackend / RetrievalWorker with the interface of the reference's ESA native
back-end (ucm/sparse/esa/retrieval/cpy/retrieval_backend.cpp:17-225 and
ucm/sparse/esa/retrieval/retrieval_worker.py:10-34), backed by the device-resident object of the
C ABI (ucmx_retrieval_*): the representative table lives in HBM, submit() enqueues the scoring and
top-k kernels on a private stream and returns at once, poll() is an event query.

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

    # -- the reference's four methods -------------------------------------------------------------
    def submit(self, query, topk: int, indexes) -> int:
        q = np.ascontiguousarray(_as_numpy(query), dtype=np.float32)
        idx = np.ascontiguousarray(_as_numpy(indexes), dtype=np.int32)
        if q.ndim != 2 or q.shape[1] != self.dim:
            raise RuntimeError("Query dim mismatch")
        if idx.ndim != 2 or idx.shape[0] != q.shape[0]:
            raise RuntimeError("Query and indexes batch mismatch")
        rid = C.c_int32(-1)
        st = N.lib.ucmx_retrieval_submit(self._h, q.ctypes.data_as(C.c_void_p), q.shape[0], q.shape[1], int(topk),
                                         idx.ctypes.data_as(C.c_void_p), idx.shape[1], C.byref(rid))
        N.check("ucmx_retrieval_submit", st, 3)   # offsets fill + score + top-k
        return rid.value

    def poll(self, req_id: int) -> bool:
        ready = C.c_int32(0)
        N.check("ucmx_retrieval_poll", N.lib.ucmx_retrieval_poll(self._h, req_id, C.byref(ready)), 0)
        return bool(ready.value)

    def wait(self, req_id: int) -> None:
        st = N.lib.ucmx_retrieval_wait(self._h, req_id)
        if st == N.ENOOBJ:
            raise RuntimeError("Bad req_id")
        N.check("ucmx_retrieval_wait", st, 0)

    def get_result(self, req_id: int) -> dict:
        b, k = C.c_int32(0), C.c_int32(0)
        st = N.lib.ucmx_retrieval_result_shape(self._h, req_id, C.byref(b), C.byref(k))
        if st == N.ENOOBJ:
            raise RuntimeError("Result not ready")
        N.check("ucmx_retrieval_result_shape", st, 0)
        indices = np.empty((b.value, k.value), np.int32)
        scores = np.empty((b.value, k.value), np.float32)
        st = N.lib.ucmx_retrieval_get_result(self._h, req_id, indices.ctypes.data_as(C.c_void_p),
                                             scores.ctypes.data_as(C.c_void_p))
        if st == N.ENOOBJ:
            raise RuntimeError("Result not ready")
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
