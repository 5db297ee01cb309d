"""Layer-wise KV connector: stored-block offsets against the reference's own DataOffset (executed from
the text of uc_connector.py when a checkout is present, and against recorded values always), and the
batching logic on a fake store.  No GPU needed."""
import ast
import os
import types

import numpy as np
import pytest
import torch

from ucmx.connector import ReqMeta, UCConnectorV1Metadata, UnifiedCacheConnectorV1, _extract_layer_index
from ucmx.store.ucmstore import Task, UcmKVStoreBase

from oracle import oracle as _orc  # noqa: E402

REF = _orc.reference_root() or ""
REF_FILE = os.path.join(REF, "ucm", "integration", "vllm", "uc_connector.py")

# (tp, rank, layer, is_v, is_mla) -> offset, recorded from the reference's DataOffset for a
# [2, 4, 16, 2, 8] bf16 layer (MLA: [4, 16, 8])
RECORDED = {(1, 0, 0, False, False): 0, (1, 0, 0, True, False): 512, (1, 0, 3, False, False): 3072, (1, 0, 3, True, False): 3584,
            (2, 1, 0, False, False): 1024, (2, 1, 2, True, False): 5632, (4, 3, 5, False, False): 23552,
            (4, 2, 1, True, False): 6656, (1, 0, 4, False, True): 1024, (2, 1, 4, False, True): 1024}


def fake_config(tp=1, layers=4, heads=2, head_size=8, block=16, mla=False, extra=None, kv_role="kv_both"):
    mc = types.SimpleNamespace(dtype=torch.bfloat16, is_deepseek_mla=mla, get_num_layers=lambda pc: layers,
                               get_num_kv_heads=lambda pc: heads, get_head_size=lambda: head_size)
    return types.SimpleNamespace(model_config=mc, parallel_config=types.SimpleNamespace(tensor_parallel_size=tp),
                                 cache_config=types.SimpleNamespace(block_size=block),
                                 kv_transfer_config=types.SimpleNamespace(kv_role=kv_role, kv_connector_extra_config=extra or {}))


class FakeStore(UcmKVStoreBase):
    """Records submissions; moves nothing."""

    def __init__(self, fail=()):
        super().__init__({})
        self.calls, self.waits, self.fail = [], [], set(fail)

    def cc_store(self): return 0
    def create(self, ids): return [0] * len(ids)
    def lookup(self, ids): return [False] * len(ids)
    def prefetch(self, ids): pass
    def load(self, ids, off, t): raise AssertionError("the batched connector describes transfers by address")
    def dump(self, ids, off, t): raise AssertionError("the batched connector describes transfers by address")

    def _task(self, kind, ids, off, addr, size):
        t = Task()
        t.n = len(self.calls)
        self.calls.append((kind, list(ids), list(off), list(addr), list(size)))
        return t

    def fetch_data(self, ids, off, addr, size): return self._task("load", ids, off, addr, size)
    def dump_data(self, ids, off, addr, size): return self._task("dump", ids, off, addr, size)

    def wait(self, task):
        self.waits.append(task.n)
        assert self.waits.count(task.n) == 1, "a task must be waited on once"
        return -1 if task.n in self.fail else 0

    def commit(self, ids, ok=True): pass
    def check(self, task): return 0, True


def kv_layer(mla=False):
    return torch.zeros((4, 16, 8), dtype=torch.bfloat16) if mla else torch.zeros((2, 4, 16, 2, 8), dtype=torch.bfloat16)


def test_data_offset_matches_recorded_reference_values():
    for (tp, rank, layer, is_v, mla), want in RECORDED.items():
        c = UnifiedCacheConnectorV1(fake_config(tp=tp, mla=mla), "worker", rank=rank, store=FakeStore())
        assert c.DataOffset(kv_layer(mla), rank, layer, is_v) == want


@pytest.mark.skipif(not os.path.exists(REF_FILE), reason="no UCM checkout")
def test_data_offset_matches_reference_function_text():
    src = open(REF_FILE).read()
    cls = [n for n in ast.parse(src).body if isinstance(n, ast.ClassDef) and n.name == "UnifiedCacheConnectorV1"][0]
    fn = [n for n in cls.body if isinstance(n, ast.FunctionDef) and n.name == "DataOffset"][0]
    ns = {"logger": types.SimpleNamespace(debug=lambda *a, **k: None)}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), "uc_connector.DataOffset", "exec"), ns)
    rng = np.random.default_rng(0)
    for _ in range(200):
        tp = int(rng.choice([1, 2, 4, 8]))
        rank, layer, is_v, mla = int(rng.integers(0, tp)), int(rng.integers(0, 40)), bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        me = types.SimpleNamespace(total_tp_size=tp, is_mla=mla, rank=rank)
        me.DataOffset = lambda kv, r, l, v, me=me: ns["DataOffset"](me, kv, r, l, v)
        want = ns["DataOffset"](me, kv_layer(mla), rank, layer, is_v and not mla)
        c = UnifiedCacheConnectorV1(fake_config(tp=tp, mla=mla), "worker", rank=rank, store=FakeStore())
        assert c.DataOffset(kv_layer(mla), rank, layer, is_v and not mla) == want
        if (tp, rank, layer, is_v, mla) in RECORDED:
            assert want == RECORDED[(tp, rank, layer, is_v, mla)]


def test_store_sizes_follow_the_reference_formula(tmp_path):
    extra = {"ucm_connector_name": "UcmNfsStore", "ucm_connector_config": {"storage_backends": str(tmp_path)}}
    c = UnifiedCacheConnectorV1(fake_config(tp=2, layers=4, heads=2, head_size=8, block=16, extra=extra), "scheduler")
    # kv_block_size = block * elem * head_size * layers * heads * tp * 2 (uc_connector.py:138-143), one file per block
    assert c.connector.create([b"0123456789abcdef"]) == [0]
    assert os.path.getsize(c.connector.path(b"0123456789abcdef", True)) == 16 * 2 * 8 * 4 * 2 * 2 * 2
    with pytest.raises(TypeError, match="no storage connector"):
        UnifiedCacheConnectorV1(fake_config(), "worker")
    assert _extract_layer_index("model.layers.17.self_attn.attn") == 17 and _extract_layer_index("no_digits") is None


def test_one_table_per_layer_covers_all_requests():
    store = FakeStore()
    c = UnifiedCacheConnectorV1(fake_config(layers=3), "worker", store=store)
    caches = {f"model.layers.{l}.attn": kv_layer() for l in range(3)}
    c.register_kv_caches(caches)
    meta = UCConnectorV1Metadata([ReqMeta("a", load_blocks=[("h1", 3), ("h2", 0)]), ReqMeta("b", load_blocks=[("h3", 1)]),
                                  ReqMeta("c", dump_blocks=[("h4", 2)])])
    c.bind_connector_metadata(meta)
    c.start_load_kv()
    assert len(store.calls) == 3                                   # one submission per layer, not per request and K/V
    kind, ids, off, addr, size = store.calls[1]
    layer = caches["model.layers.1.attn"]
    assert kind == "load" and ids == ["h1", "h2", "h3"] * 2
    k_off, v_off = c.DataOffset(layer, 0, 1, False), c.DataOffset(layer, 0, 1, True)
    assert off == [k_off] * 3 + [v_off] * 3 and size == [512] * 6
    want = [layer[0][b].data_ptr() for b in (3, 0, 1)] + [layer[1][b].data_ptr() for b in (3, 0, 1)]
    assert addr == want                                              # the same addresses the per-block tensor views have
    tensors, offsets = c.get_tensor_and_offset_layerwise([3, 0, 1], layer, "model.layers.1.attn")
    assert [t.data_ptr() for t in tensors] == want and offsets == off
    for name in caches:
        c.wait_for_layer_load(name)
    assert sorted(store.waits) == [0, 1, 2] and not c.get_block_ids_with_load_errors()
    # dumps: one submission per layer, every block of every request listed under the request
    for name, layer in caches.items():
        c.save_kv_layer(name, layer)
    assert [k for k, *_ in store.calls[3:]] == ["dump"] * 3 and store.calls[3][1] == ["h4", "h4"]
    assert c.wait_for_save() == {"c": ["h4"]}


def test_failed_batch_marks_every_participant():
    store = FakeStore(fail={1})
    c = UnifiedCacheConnectorV1(fake_config(layers=2), "worker", store=store)
    caches = {f"layers.{l}": kv_layer() for l in range(2)}
    c.register_kv_caches(caches)
    c.bind_connector_metadata(UCConnectorV1Metadata([ReqMeta("a", load_blocks=[("h1", 3)]), ReqMeta("b", load_blocks=[("h2", 1)])]))
    c.start_load_kv()
    c.wait_for_layer_load("layers.0")
    assert not c.get_block_ids_with_load_errors()
    c.wait_for_layer_load("layers.1")
    assert c.get_block_ids_with_load_errors() == {3, 1}
    c.clear_connector_metadata()
    # asynchronous loads are polled through get_finished
    store2 = FakeStore()
    c2 = UnifiedCacheConnectorV1(fake_config(layers=2), "worker", store=store2)
    c2.register_kv_caches(caches)
    c2.bind_connector_metadata(UCConnectorV1Metadata([ReqMeta("x", load_blocks=[("h1", 2)], load_async=True),
                                                      ReqMeta("y", load_blocks=[("h5", 0)], load_async=True)]))
    c2.start_load_kv()
    assert c2.layerwise_load_tasks == {} and len(store2.calls) == 2
    assert c2.get_finished(set()) == (None, {"x", "y"}) and sorted(store2.waits) == [0, 1]
    assert c2.get_finished(set()) == (None, set())
    # a consumer never dumps
    c3 = UnifiedCacheConnectorV1(fake_config(layers=2, kv_role="kv_consumer"), "worker", store=FakeStore())
    c3.bind_connector_metadata(UCConnectorV1Metadata([ReqMeta("c", dump_blocks=[("h4", 2)])]))
    c3.save_kv_layer("layers.0", kv_layer())
    assert c3.wait_for_save() is None and c3.connector.calls == []
