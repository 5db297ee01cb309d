"""The decode-step engine's three ways of running a step - call by call with device inputs, end to end with pinned
host buffers on two streams, and the same replayed from one CUDA graph - must select the same blocks; the graph
must pick up queries written into the pinned buffer after it was captured."""
import numpy as np
import pytest
import torch

import helpers as H_

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def make_engine(overlap=False):
    from ucmx.engine import DecodeRetrievalEngine
    from ucmx.workloads import KvShape, ragged_decode_batch
    shape = KvShape(n_q_heads=32, n_kv_heads=8, head_dim=128, block_tokens=128, n_layers=3)
    batch = ragged_decode_batch(seed=31, n_req=6, min_ctx=2048, max_ctx=8192, ratio=0.1, min_k=4)
    return DecodeRetrievalEngine(shape, batch, DEV, with_kv_pool=True, overlap=overlap)


def test_selection_on_a_second_stream_changes_nothing():
    """Scoring and top-k of layer l+1 on a stream of their own beside layer l's block moves: the same selections and
    the same gathered blocks as layer by layer, call by call and replayed from the captured graph."""
    from ucmx.engine import DecodeRetrievalEngine
    from ucmx.workloads import KvShape, ragged_decode_batch
    shape = KvShape(n_q_heads=32, n_kv_heads=8, head_dim=128, block_tokens=128, n_layers=3)
    batch = ragged_decode_batch(seed=31, n_req=6, min_ctx=2048, max_ctx=8192, ratio=0.1, min_k=4)
    plain = DecodeRetrievalEngine(shape, batch, DEV, with_kv_pool=True, seed=9)
    plain.make_queries()
    plain.step()
    torch.cuda.synchronize()
    eng = DecodeRetrievalEngine(shape, batch, DEV, with_kv_pool=True, seed=9, overlap=True)
    eng.make_queries()
    assert torch.equal(eng.q_dev, plain.q_dev)
    for replay in (False, True, True):
        if replay and eng.graph is None:
            eng.capture()
        eng.sel_ids.fill_(-7)
        eng.staging.zero_()
        eng.step()
        torch.cuda.synchronize()
        assert torch.equal(eng.sel_ids, plain.sel_ids) and torch.equal(eng.sel_counts, plain.sel_counts)
        assert torch.equal(eng.staging, plain.staging)
    from ucmx import _native
    assert _native.device_error() == 0


def test_scoring_launched_early_behind_a_topk_changes_nothing():
    """Scoring kernels allowed to begin under the tail of the top-k ahead of them (they share the score buffer with it
    and store only after its end): same scores and same selections as plain launches, call by call and replayed from
    a graph, on a batch that fills every SM."""
    from ucmx import _native, ops
    from ucmx.workloads import ragged_decode_batch
    batch = ragged_decode_batch(seed=77, n_req=48, min_ctx=16384, max_ctx=65536, ratio=0.1, min_k=4)
    g = torch.Generator(device=DEV).manual_seed(77)
    H, D, n_tab = 8, 128, 4
    off = torch.from_numpy(batch.offsets).to(DEV)
    table = torch.from_numpy(batch.block_table).to(DEV)
    kk = torch.from_numpy(batch.k_per_req).to(DEV)
    reps = [(torch.randn((batch.n_slots, H, 1, D), generator=g, device=DEV) * 0.09).to(torch.bfloat16) for _ in range(n_tab)]
    q = torch.randn((n_tab, batch.n_req, 32, D), generator=g, device=DEV).to(torch.bfloat16)
    stride = int(batch.k_per_req.max())
    scores = torch.empty((batch.total,), dtype=torch.float32, device=DEV)

    qbar = [ops.query_group_mean(q[i], H) for i in range(n_tab)]     # (made ahead of time: an early launch may not read
    torch.cuda.synchronize()                                          #  what the kernel in front of it writes)

    def run(early, ids, vals, kept):
        for i in range(n_tab):
            if i % 2 == 0:
                ops.score_dot_query(reps[i], off, q[i], total=batch.total, slot_ids=table, n_kv_heads=H, out=scores,
                                    early=early and i > 0)
            else:                                                     # the two-call form, fp32 queries
                ops.score_dot(reps[i], off, qbar[i], total=batch.total, slot_ids=table, n_kv_heads=H, head_dim=D,
                              out=scores, early=early)
            if kept is not None:
                kept[i].copy_(scores)
            ops.topk_ragged(scores, off, kk, out_stride=stride, id_map=table, out_idx=ids[i], out_scores=vals[i])

    def fresh():
        return (torch.full((n_tab, batch.n_req, stride), -7, dtype=torch.int32, device=DEV),
                torch.zeros((n_tab, batch.n_req, stride), dtype=torch.float32, device=DEV))

    want_ids, want_vals = fresh()
    want_scores = torch.empty((n_tab, batch.total), dtype=torch.float32, device=DEV)
    run(False, want_ids, want_vals, want_scores)
    torch.cuda.synchronize()
    got_ids, got_vals = fresh()
    got_scores = torch.empty_like(want_scores)
    run(True, got_ids, got_vals, got_scores)
    torch.cuda.synchronize()
    assert torch.equal(got_scores, want_scores)
    assert torch.equal(got_ids, want_ids) and torch.equal(got_vals, want_vals)

    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run(True, got_ids, got_vals, None)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run(True, got_ids, got_vals, None)
    for _ in range(4):
        got_ids.fill_(-7)
        got_vals.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(got_ids, want_ids) and torch.equal(got_vals, want_vals)
    assert _native.device_error() == 0


def test_multi_representative_scoring_launched_early(oracle):
    """The row-ring kernel with two representatives per head, launched early behind a top-k that still reads the score
    buffer, replayed from a graph: the scores of the CPU checker, every time."""
    from ucmx import ops
    from ucmx.workloads import ragged_decode_batch
    batch = ragged_decode_batch(seed=78, n_req=24, min_ctx=8192, max_ctx=32768, ratio=0.1, min_k=4)
    rng = np.random.default_rng(78)
    Hkv, R, D, n_tab = 8, 2, 128, 3
    reps16 = [H_.randn_bf16(rng, (batch.n_slots, Hkv, R, D), 0.09) for _ in range(n_tab)]
    q = H_.bf16_to_f32(H_.randn_bf16(rng, (batch.n_req, Hkv * D)))
    want = [oracle.score_dot_gsa(H_.bf16_to_f32(r), Hkv, R, D, batch.offsets, batch.block_table, q) for r in reps16]
    bf = lambda u: torch.from_numpy(u.view(np.int16).copy()).to(DEV).view(torch.bfloat16)
    reps = [bf(r) for r in reps16]
    off = torch.from_numpy(batch.offsets).to(DEV)
    table = torch.from_numpy(batch.block_table).to(DEV)
    kk = torch.from_numpy(batch.k_per_req).to(DEV)
    qd = torch.from_numpy(q).to(DEV)
    scores = torch.empty((batch.total,), dtype=torch.float32, device=DEV)
    kept = torch.empty((n_tab, batch.total), dtype=torch.float32, device=DEV)
    stride = int(batch.k_per_req.max())

    def run():
        for i in range(n_tab):
            ops.score_dot(reps[i], off, qd, total=batch.total, slot_ids=table, n_kv_heads=Hkv, head_dim=D, n_rep=R,
                          out=scores, early=i > 0)
            kept[i].copy_(scores)
            ops.topk_ragged(scores, off, kk, out_stride=stride)

    side = torch.cuda.Stream(device=DEV)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run()
    for _ in range(3):
        kept.zero_()
        graph.replay()
        torch.cuda.synchronize()
        got = kept.cpu().numpy()
        for i in range(n_tab):
            np.testing.assert_allclose(got[i], want[i], rtol=1e-3, atol=1e-3 * float(np.abs(want[i]).std()))


@pytest.mark.parametrize("overlap", [False, True])
def test_host_step_and_its_graph_match_the_device_step(overlap):
    eng = make_engine(overlap)
    eng.make_queries()
    eng.step()
    torch.cuda.synchronize()
    want_ids, want_cnt = eng.sel_ids.cpu().numpy().copy(), eng.sel_counts.cpu().numpy().copy()
    want_staging = eng.staging.cpu().numpy().copy()

    eng.alloc_host()                       # q_host starts as a copy of the device queries
    eng.sel_ids.fill_(-7)
    got = eng.step_host()
    assert np.array_equal(got.numpy(), want_ids) and np.array_equal(eng.cnt_host.numpy(), want_cnt)

    eng.capture_host()
    assert eng.host_graph is not None
    eng.sel_host.fill_(-7)
    eng.staging.zero_()
    got = eng.step_host()                  # a replay
    assert np.array_equal(got.numpy(), want_ids) and np.array_equal(eng.cnt_host.numpy(), want_cnt)
    assert np.array_equal(eng.staging.cpu().numpy(), want_staging)     # last layer's gathered blocks

    # new queries in the pinned buffer: the replay must read them, and agree with a plain device step on them
    g = torch.Generator().manual_seed(5)
    eng.q_host.copy_(torch.randn(eng.q_host.shape, generator=g).to(torch.bfloat16))
    got = eng.step_host().numpy().copy()
    eng.host_graph = None
    eng.q_dev.copy_(eng.q_host)
    eng.step()
    torch.cuda.synchronize()
    assert np.array_equal(got, eng.sel_ids.cpu().numpy())
    assert not np.array_equal(got, want_ids)

    from ucmx import _native
    assert _native.device_error() == 0


@pytest.mark.parametrize("heads_local", [1, 2, 8])
def test_tensor_parallel_step_replays_from_a_graph(heads_local):
    """What one rank of a tensor-parallel run does (here alone, as rank 0 of a one-rank exchange): the scoring
    kernel delivers into the exchange buffer and publishes the round, the top-k kernel collects; captured once and
    replayed.  One KV head per rank takes the narrow-row kernel after a separate query-mean launch, two or more
    take the copy-engine kernel with the mean folded in.  The selections must equal the plain engine's."""
    from ucmx import _native, ops
    from ucmx.engine import DecodeRetrievalEngine
    from ucmx.parallel import PeerScoreExchange
    from ucmx.workloads import KvShape, fixed_batch
    shape = KvShape(n_q_heads=64, n_kv_heads=8, head_dim=128, block_tokens=128, n_layers=2)
    batch = fixed_batch(3, 700, 90, seed=77)
    plain = DecodeRetrievalEngine(shape, batch, DEV, with_kv_pool=False, heads_local=heads_local, seed=5,
                                  order=ops.ORDER_INDEX_ASC)
    plain.make_queries()
    plain.step()
    torch.cuda.synchronize()
    want = plain.sel_ids.cpu().numpy().copy()
    buf = torch.zeros(PeerScoreExchange.words_needed(1, batch.total), dtype=torch.float32, device=DEV)
    ex = PeerScoreExchange([buf.data_ptr()], 0, batch.total, DEV, buf)
    eng = DecodeRetrievalEngine(shape, batch, DEV, with_kv_pool=False, heads_local=heads_local, seed=5,
                                peer_exchange=ex, order=ops.ORDER_INDEX_ASC)
    eng.make_queries()                                     # the same seed: the same tables and queries
    eng.capture()
    for _ in range(3):                                     # odd and even rounds
        eng.sel_ids.fill_(-7)
        eng.step()
        torch.cuda.synchronize()
        assert np.array_equal(eng.sel_ids.cpu().numpy(), want)
    assert _native.device_error() == 0
