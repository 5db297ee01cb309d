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

submit / wait / get_result - three calls per request and layer in ESA's pattern - are methods of a small
CPython type (csrc/pybackend.c, built beside the library) that calls the C ABI directly, and
RetrievalWorkerBackend derives from it; the other methods go through ctypes.
"""
from __future__ import annotations

import ctypes as C
import importlib.util
import os

import numpy as np

from . import _native as N


def _load_fast():
    """The CPython front of ucmx_retrieval_* (built by build.py next to libucmx.so), bound to the loaded library."""
    lib_dir = os.path.dirname(N.LIB_PATH)
    names = [f for f in os.listdir(lib_dir) if f.startswith("_ucmx_fast") and f.endswith(".so")] if os.path.isdir(lib_dir) else []
    if not names:
        raise ImportError(f"_ucmx_fast is missing from {lib_dir}: run unified-cache-management_b200/build.py")
    spec = importlib.util.spec_from_file_location("_ucmx_fast", os.path.join(lib_dir, sorted(names)[0]))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    addr = lambda fn: C.cast(fn, C.c_void_p).value   # noqa: E731
    mod.bind(addr(N.lib.ucmx_retrieval_submit), addr(N.lib.ucmx_retrieval_wait), addr(N.lib.ucmx_retrieval_get_result),
             addr(N.lib.ucmx_retrieval_result_shape), _raise_status)
    return mod


def _raise_status(fn_name: str, status: int) -> None:
    raise N.UcmxError(fn_name, status, N.last_error())


_fast = _load_fast()


class RetrievalWorkerBackend(_fast.Backend):
    """submit(query float32 [b, dim], topk, indexes int32 [b, max_idx], -1 = pad) -> req_id; wait(req_id);
    get_result(req_id) -> {"indices": int32 [b, k], "scores": float32 [b, k]} are inherited from the C type; poll,
    flush and the rest are below."""

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
        _fast.Backend.__init__(self, self._h.value, self.dim)

    def _submit_converted(self, query, topk, indexes) -> int:
        """Called by submit for anything that is not a plain C-contiguous float32 / int32 numpy array."""
        q = np.ascontiguousarray(_as_numpy(query), dtype=np.float32)
        idx = np.ascontiguousarray(_as_numpy(indexes), dtype=np.int32)
        if q.ndim != 2 or q.shape[1] != self.dim:
            raise RuntimeError("Query dim mismatch")
        if idx.ndim != 2 or idx.shape[0] != q.shape[0]:
            raise RuntimeError("Query and indexes batch mismatch")
        return self.submit(q, int(topk), idx)

    def flush(self) -> None:
        """Send everything submitted so far to the GPU now (otherwise the first poll/wait/get_result does it)."""
        N.check("ucmx_retrieval_flush", N.lib.ucmx_retrieval_flush(self._h), 0)

    def poll(self, req_id: int) -> bool:
        ready = C.c_int32(0)
        N.check("ucmx_retrieval_poll", N.lib.ucmx_retrieval_poll(self._h, req_id, C.byref(ready)), 0)
        return bool(ready.value)

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
            _fast.Backend.__init__(self, 0, self.dim)      # the C side forgets the handle too

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
