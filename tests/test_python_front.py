"""The CPython front of the retrieval object (csrc/pybackend.c): it is built beside the library, binds to the
library's entry points, and reports the reference's shape errors with the reference's words - all without a GPU
(no call below reaches the device)."""
import numpy as np
import pytest


def test_front_is_built_and_bound():
    from ucmx import retrieval
    assert retrieval._fast.__name__ == "_ucmx_fast"
    fb = retrieval._fast.Backend(0, 16)
    for name in ("submit", "wait", "get_result"):
        assert callable(getattr(fb, name))


def test_shape_errors_and_conversion_requests():
    from ucmx import retrieval
    fb = retrieval._fast.Backend(0, 16)
    q, idx = np.zeros((2, 16), np.float32), np.zeros((2, 5), np.int32)
    # arrays the C side cannot read as they are: the caller converts first (None), nothing is raised
    assert fb.submit(q.astype(np.float64), 3, idx) is None
    assert fb.submit(q, 3, idx.astype(np.int64)) is None
    assert fb.submit(np.asfortranarray(q), 3, idx) is None
    assert fb.submit(q.tolist(), 3, idx) is None
    with pytest.raises(RuntimeError, match="Query dim mismatch"):
        fb.submit(np.zeros((2, 8), np.float32), 3, idx)
    with pytest.raises(RuntimeError, match="Query and indexes batch mismatch"):
        fb.submit(q, 3, np.zeros((3, 5), np.int32))
    with pytest.raises(RuntimeError, match="Query dim mismatch"):
        fb.submit(np.zeros((16,), np.float32), 3, idx)
    assert fb.get_result(7) is None            # a request this object never saw
    assert fb.get_result(-1) is None
