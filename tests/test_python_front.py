"""The CPython front of the retrieval object (csrc/pybackend.c): it is built beside the library, binds to the
library's entry points, hands arrays it cannot read as they are to the subclass for conversion, and reports the
reference's shape errors with the reference's words - all without a GPU (no call below reaches the device)."""
import numpy as np
import pytest


def test_front_is_built_and_the_backend_derives_from_it():
    from ucmx import retrieval
    assert retrieval._fast.__name__ == "_ucmx_fast"
    assert issubclass(retrieval.RetrievalWorkerBackend, retrieval._fast.Backend)
    for name in ("submit", "wait", "get_result"):
        assert getattr(retrieval.RetrievalWorkerBackend, name) is getattr(retrieval._fast.Backend, name)


def test_shape_errors_and_conversion_requests():
    from ucmx import retrieval

    class Probe(retrieval._fast.Backend):
        def _submit_converted(self, query, topk, indexes):
            self.asked = (type(query).__name__, int(topk), getattr(indexes, "dtype", None))
            return -7

    fb = Probe(1, 16)          # a handle that is never used: every call below stops before the library
    q, idx = np.zeros((2, 16), np.float32), np.zeros((2, 5), np.int32)
    # arrays the C side cannot read as they are go to the subclass
    assert fb.submit(q.astype(np.float64), 3, idx) == -7 and fb.asked[1] == 3
    assert fb.submit(q, 3, idx.astype(np.int64)) == -7 and fb.asked[2] == np.int64
    assert fb.submit(np.asfortranarray(q), 3, idx) == -7
    assert fb.submit(q.tolist(), 3, idx) == -7 and fb.asked[0] == "list"
    with pytest.raises(RuntimeError, match="Query dim mismatch"):
        fb.submit(np.zeros((2, 8), np.float32), 3, idx)
    with pytest.raises(RuntimeError, match="Query and indexes batch mismatch"):
        fb.submit(q, 3, np.zeros((3, 5), np.int32))
    with pytest.raises(RuntimeError, match="Query dim mismatch"):
        fb.submit(np.zeros((16,), np.float32), 3, idx)
    with pytest.raises(RuntimeError, match="Result not ready"):
        fb.get_result(7)           # a request this object never saw
    with pytest.raises(RuntimeError, match="Result not ready"):
        fb.get_result(-1)
    closed = Probe(0, 16)
    with pytest.raises(RuntimeError, match="closed"):
        closed.submit(q, 3, idx)
    with pytest.raises(RuntimeError, match="closed"):
        closed.wait(0)
