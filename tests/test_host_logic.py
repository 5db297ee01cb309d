"""Host-side logic of the reference-facing layers that needs no GPU: registries, slot pool, block
hashes, the scheduler-side estimates of ESA, GSA's top-k length rule, store offsets."""
import os
from types import SimpleNamespace

import numpy as np
import pytest

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def cfg(method="ESA", extra=None):
    model = SimpleNamespace(max_model_len=4096, hf_config=SimpleNamespace(num_hidden_layers=4),
                            get_num_kv_heads=lambda pc: 8, get_head_size=lambda: 128)
    d = {"init_window_sz": 1, "local_window_sz": 2, "min_blocks": 4, "sparse_ratio": 0.3, "retrieval_stride": 5}
    d.update(extra or {})
    return SimpleNamespace(parallel_config=SimpleNamespace(rank=0, tensor_parallel_size=1),
                           cache_config=SimpleNamespace(block_size=128), model_config=model,
                           scheduler_config=SimpleNamespace(max_num_seqs=8),
                           kv_transfer_config=SimpleNamespace(kv_connector_extra_config={"ucm_sparse_config": {method: d}}))


def test_factory_and_state_registry():
    from ucmx.sparse import state
    from ucmx.sparse.base import UcmSparseBase, UcmSparseRole
    from ucmx.sparse.esa import ESA
    from ucmx.sparse.factory import UcmSparseFactory
    from ucmx.store.factory import UcmConnectorFactory
    state.reset_ucm_sparse()
    assert not state.has_ucm_sparse()
    with pytest.raises(RuntimeError):
        state.get_ucm_sparse()
    state.ensure_ucm_sparse_initialized(cfg(), UcmSparseRole.SCHEDULER)
    agent = state.get_ucm_sparse()
    assert isinstance(agent, ESA) and isinstance(agent, UcmSparseBase) and agent.role == UcmSparseRole.SCHEDULER
    state.ensure_ucm_sparse_initialized(cfg(), UcmSparseRole.WORKER)        # second call keeps the first agent
    assert state.get_ucm_sparse() is agent
    state.reset_ucm_sparse()
    with pytest.raises(ValueError):
        UcmSparseFactory.create_sparse_method(cfg("Nope"), UcmSparseRole.SCHEDULER)
    with pytest.raises(ValueError):
        UcmSparseFactory.register_sparse_method("ESA", "x", "y")
    with pytest.raises(ValueError):
        UcmConnectorFactory.create_connector("UcmNoStore", {})


def test_repre_pool_and_block_hashes():
    from ucmx.sparse.esa import ReprePool, block_hashes_of, sparse_prefill_range
    p = ReprePool(10)
    a = p.allocate(4)
    b = p.allocate(3)
    assert a == [0, 1, 2, 3] and b == [4, 5, 6] and p.allocated == set(range(7))
    p.free(a)
    assert p.allocated == {4, 5, 6} and len(p.free_slots) == 7
    with pytest.raises(AssertionError):
        p.allocate(8)
    toks = list(range(300))
    h = block_hashes_of(toks, 128)
    assert len(h) == 2 and h[0] != h[1] and h == block_hashes_of(toks, 128)
    assert block_hashes_of(toks[:128] + [7] * 172, 128)[0] == h[0]           # same first block, same hash
    assert block_hashes_of([1] + toks[1:], 128)[1] != h[1]                   # the chain carries the parent
    assert sparse_prefill_range(20 * 128, 128, 2) == 18
    assert sparse_prefill_range(33 * 128 + 5, 128, 2) == 32


def test_esa_scheduler_side():
    from ucmx.sparse.base import INVALID_SLOT, UcmSparseRole
    from ucmx.sparse.esa import ESA
    esa = ESA(cfg(), UcmSparseRole.SCHEDULER)
    req = SimpleNamespace(num_output_tokens=0, num_prompt_tokens=2560, prompt_token_ids=[0] * 2560, request_id="r")
    assert esa.estimate_num_slots_sparsed(req) == INVALID_SLOT               # still in prefill
    req.num_output_tokens = 3
    assert esa.estimate_num_slots_sparsed(req) == int(18 * 0.3) * 128 + 128 * 2 + 3
    req2 = SimpleNamespace(num_output_tokens=1, num_prompt_tokens=33 * 128 + 5, prompt_token_ids=[0] * (33 * 128 + 5))
    assert esa.estimate_num_slots_sparsed(req2) == int(32 * 0.3) * 128 + 5 + 128 + 1
    short = SimpleNamespace(num_output_tokens=1, num_prompt_tokens=100, prompt_token_ids=[0] * 100)
    assert esa.estimate_num_slots_sparsed(short) == INVALID_SLOT             # below min_blocks

    class Pool:
        def __init__(self): self.freed, self.evicted = [], []
        def _maybe_evict_cached_block(self, b): self.evicted.append(b)
        def free_blocks(self, bs): self.freed.extend(bs)
        def get_num_free_blocks(self): return 100

    class Coord:
        def __init__(self): self.single_type_managers = [SimpleNamespace(req_to_blocks={})]; self.alloc = None
        def get_blocks(self, rid): return [list(range(20))]
        def get_num_blocks_to_allocate(self, request_id, num_tokens, new_computed_blocks): return 1
        def allocate_new_blocks(self, rid, n): self.alloc = (rid, n)

    pool, coord = Pool(), Coord()
    kept = esa.allocate_slots(req, 5 * 128 + 2 * 128 + 3, coord, pool, [None])
    assert kept == list(range(12, 20)) and pool.freed == list(range(12)) and len(pool.evicted) == 20
    assert coord.single_type_managers[0].req_to_blocks["r"] == kept and coord.alloc == ("r", 5 * 128 + 2 * 128 + 3)


def test_gsa_topk_len_and_store_offsets():
    from ucmx.sparse.gsa import compute_topk_len
    from ucmx.store.dramstore import store_offset
    assert [compute_topk_len(n) for n in (10, 32, 100, 120, 160, 1000)] == [10, 32, 32, 36, 48, 48]
    for rank, tp, layer, is_v, want in G["offset_cases"]:
        assert store_offset((128, 8 // tp, 128), int(rank), int(tp), 2, int(layer), bool(is_v)) == want


def test_workloads_are_seeded_and_in_range():
    from ucmx.workloads import ragged_decode_batch
    a, b = ragged_decode_batch(seed=2002), ragged_decode_batch(seed=2002)
    assert np.array_equal(a.blocks_per_req, b.blocks_per_req) and np.array_equal(a.block_table, b.block_table)
    assert a.n_req == 64 and a.blocks_per_req.min() >= 64 and a.blocks_per_req.max() <= 1024
    assert (a.k_per_req == np.maximum(16, np.ceil(0.05 * a.blocks_per_req - 1e-9))).all()
    assert sorted(a.block_table.tolist()) == list(range(a.total))
    # the same request lengths over another block table: what every rank of a request-parallel run holds
    c = ragged_decode_batch(seed=2002, table_seed=7008)
    assert np.array_equal(a.blocks_per_req, c.blocks_per_req) and np.array_equal(a.k_per_req, c.k_per_req)
    assert not np.array_equal(a.block_table, c.block_table) and sorted(c.block_table.tolist()) == list(range(a.total))


def test_kvstar_module_rejects_bad_shapes_like_the_reference():
    """The shape checks of KVStar::Execute (simd_compute_kernel.cpp:637-666) come before any device work."""
    import torch
    from ucmx import kvstar
    q = torch.zeros((8, 32, 128), dtype=torch.float16)
    reps = torch.zeros((10, 64, 8, 32), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="Query shape must be 3D"):
        kvstar.AsyncRetrieveByCPU(q[0], reps, None, 4)
    with pytest.raises(RuntimeError, match="BlockRep shape must be 4D"):
        kvstar.AsyncRetrieveByCPU(q, reps[0], None, 4)
    with pytest.raises(RuntimeError, match="divisible"):
        kvstar.AsyncRetrieveByCPU(q[:, :30], reps, None, 4)
    with pytest.raises(RuntimeError, match="inconsistent"):
        kvstar.AsyncRetrieveByCPU(q, reps, torch.zeros((8, 16), dtype=torch.int64), 4)
    with pytest.raises(RuntimeError, match="Dimension mismatch"):
        kvstar.AsyncRetrieveByCPU(q, reps, None, 4)
    assert kvstar.GetTaskResult(123456) is None and kvstar.Wait(123456) == -1 and kvstar.Setup() == 0


def test_numa_helpers_read_sysfs_layout(tmp_path):
    from ucmx.store import numa
    dev = tmp_path / "bus" / "pci" / "devices" / "0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-19,48,50-51\n")
    assert numa.device_numa_node("0000:1B:00.0", str(tmp_path)) == 1
    assert numa.node_cpus(1, str(tmp_path)) == [16, 17, 18, 19, 48, 50, 51]
    assert numa.device_numa_node("0000:ff:00.0", str(tmp_path)) is None and numa.node_cpus(7, str(tmp_path)) == []
    (dev / "numa_node").write_text("-1\n")
    assert numa.device_numa_node("0000:1b:00.0", str(tmp_path)) is None


def test_kvstar_multistep_registered_and_slot_estimate():
    """The fourth sparse method of the reference's factory (ucm/sparse/factory.py:47-52) and its scheduler-side
    slot estimate (multistep.py:775-814): prefill is not sparsified; in decode the middle of the prompt shrinks to
    ceil(ratio * middle blocks) while the init window, the local window and everything after the prompt stay."""
    from types import SimpleNamespace as NS

    from ucmx.sparse.base import INVALID_SLOT, UcmSparseRole
    from ucmx.sparse.factory import UcmSparseFactory
    from ucmx.sparse.kvstar import KVStarMultiStep
    agent = UcmSparseFactory.create_sparse_method(cfg("KVStarMultiStep", {"sparse_ratio": 0.25}), UcmSparseRole.SCHEDULER)
    assert isinstance(agent, KVStarMultiStep)
    bs = agent.block_size
    assert agent.d_pruned == round(agent.head_size * 0.25) and agent.stride == 5 and agent.merge == 2
    assert agent.estimate_num_slots_sparsed(NS(num_output_tokens=0, num_prompt_tokens=40 * bs, num_tokens=40 * bs)) == INVALID_SLOT
    # 40 full prompt blocks: 1 + 2 stay, ceil(37 / 4) = 10 of the middle are kept -> 13 blocks, plus the decode tail
    req = NS(num_output_tokens=3, num_prompt_tokens=40 * bs, num_tokens=40 * bs + 3)
    assert agent.estimate_num_slots_sparsed(req) == 13 * bs + 3
    req = NS(num_output_tokens=bs, num_prompt_tokens=40 * bs, num_tokens=41 * bs)
    assert agent.estimate_num_slots_sparsed(req) == 14 * bs
    # a prompt no longer than the windows is left alone
    req = NS(num_output_tokens=1, num_prompt_tokens=2 * bs, num_tokens=2 * bs + 1)
    assert agent.estimate_num_slots_sparsed(req) == 2 * bs + 1
