"""The RetrievalWorkerBackend drop-in against the compiled reference's recorded answers."""
import os

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


@pytest.mark.parametrize("table_dtype", ["bf16", "f32"])
def test_backend_matches_reference(table_dtype):
    from ucmx.retrieval import RetrievalWorker, RetrievalWorkerBackend
    data, query, idx, topk = H.case_esa()
    worker = RetrievalWorker(RetrievalWorkerBackend(data, table_dtype=table_dtype))
    rid = worker.submit(query, topk, idx)
    worker.wait(rid)
    assert worker.poll(rid)
    res = worker.get_result(rid)
    assert res["indices"].shape == (3, topk) and res["scores"].dtype == np.float32
    # identical index sets and order (no ties in this case), scores to 1e-3 of the score scale
    assert np.array_equal(res["indices"], G["esa_indices"])
    np.testing.assert_allclose(res["scores"], G["esa_scores"], rtol=1e-3, atol=1e-3 * np.abs(G["esa_scores"]).mean())
    with pytest.raises(RuntimeError, match="Result not ready"):
        worker.get_result(rid)                     # results are handed out once, as in the reference
    with pytest.raises(RuntimeError, match="Bad req_id"):
        worker.wait(12345)
    with pytest.raises(RuntimeError, match="Query dim mismatch"):
        worker.submit(query[:, :512], topk, idx)
    with pytest.raises(RuntimeError, match="batch mismatch"):
        worker.submit(query, topk, idx[:2])


def test_backend_short_rows_update_and_many_requests(oracle):
    from ucmx.retrieval import RetrievalWorkerBackend
    rng = np.random.default_rng(61)
    data = H.bf16_to_f32(H.randn_bf16(rng, (500, 256), 0.1))
    be = RetrievalWorkerBackend(data)
    new_rows = H.bf16_to_f32(H.randn_bf16(rng, (3, 256), 0.1))
    be.update_rows([10, 499, 0], new_rows)
    data[[10, 499, 0]] = new_rows
    rids, cases = [], []
    for i in range(5):
        b = 1 + i
        q = H.bf16_to_f32(H.randn_bf16(rng, (b, 256)))
        idx = np.full((b, 40), -1, np.int32)
        for r in range(b):
            n = int(rng.integers(1, 41))
            idx[r, :n] = rng.permutation(500)[:n]
        rids.append(be.submit(q, 8, idx))
        cases.append((q, idx))
    for rid, (q, idx) in zip(rids, cases):
        be.wait(rid)
        res = be.get_result(rid)
        for r in range(len(q)):
            allowed = idx[r][idx[r] >= 0]
            s = oracle.score_dot_esa(data, np.array([0, len(allowed)], np.int32), allowed, q[r:r + 1])
            wi, ws = oracle.topk_esa(s, 8, allowed)
            m = len(wi)
            assert np.array_equal(res["indices"][r, :m], wi)
            assert (res["indices"][r, m:] == -1).all() and np.isneginf(res["scores"][r, m:]).all()
    be.close()


def test_twenty_thousand_requests_outstanding(oracle):
    """More requests in flight than the object's slot table (16 384) and the Python front's shape table (8 192)
    hold: the overflow paths give the same answers, in any order of collection."""
    from ucmx.retrieval import RetrievalWorkerBackend
    rng = np.random.default_rng(62)
    data = H.bf16_to_f32(H.randn_bf16(rng, (64, 32), 0.1))
    be = RetrievalWorkerBackend(data)
    n = 20_000
    q = H.bf16_to_f32(H.randn_bf16(rng, (n, 32)))
    idx = np.stack([rng.permutation(64)[:6] for _ in range(n)]).astype(np.int32)
    rids = [be.submit(q[i:i + 1], 2 + i % 3, idx[i:i + 1]) for i in range(n)]
    assert len(set(rids)) == n
    order = rng.permutation(n)
    check = set(order[:300].tolist()) | {0, 8191, 8192, 16383, 16384, n - 1}
    for i in order:
        be.wait(rids[i])
        res = be.get_result(rids[i])
        k = 2 + i % 3
        assert res["indices"].shape == (1, k)
        if int(i) in check:
            s = oracle.score_dot_esa(data, np.array([0, 6], np.int32), idx[i], q[i:i + 1])
            wi, _ = oracle.topk_esa(s, k, idx[i])
            assert np.array_equal(res["indices"][0], wi)
    with pytest.raises(RuntimeError, match="Result not ready"):
        be.get_result(rids[0])
    be.close()
