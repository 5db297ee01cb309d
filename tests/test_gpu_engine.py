"""The decode-step engine's three ways of running a step - call by call with device inputs, end to end with pinned
host buffers on two streams, and the same replayed from one CUDA graph - must select the same blocks; the graph
must pick up queries written into the pinned buffer after it was captured."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def make_engine():
    from ucmx.engine import DecodeRetrievalEngine
    from ucmx.workloads import KvShape, ragged_decode_batch
    shape = KvShape(n_q_heads=32, n_kv_heads=8, head_dim=128, block_tokens=128, n_layers=3)
    batch = ragged_decode_batch(seed=31, n_req=6, min_ctx=2048, max_ctx=8192, ratio=0.1, min_k=4)
    return DecodeRetrievalEngine(shape, batch, DEV, with_kv_pool=True)


def test_host_step_and_its_graph_match_the_device_step():
    eng = make_engine()
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
