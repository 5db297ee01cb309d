"""Layer-wise KV connector on the GPU: blocks dumped layer by layer come back bit-identical into other
cache slots, through both stores, and the batched submissions leave exactly the bytes in the store
that the reference's per-block call pattern (one `dump` per block, layer and K/V) leaves."""
import os
import types

import numpy as np
import pytest
import torch

from ucmx import _native as N
from ucmx.connector import ReqMeta, UCConnectorV1Metadata, UnifiedCacheConnectorV1
from ucmx.store.dramstore import UcmDramStore
from ucmx.store.nfsstore import UcmNfsStore

pytestmark = pytest.mark.gpu
L, NB, T, H, D = 3, 24, 16, 2, 64


def fake_config(extra):
    mc = types.SimpleNamespace(dtype=torch.bfloat16, is_deepseek_mla=False, get_num_layers=lambda pc: L,
                               get_num_kv_heads=lambda pc: H, get_head_size=lambda: D)
    return types.SimpleNamespace(model_config=mc, parallel_config=types.SimpleNamespace(tensor_parallel_size=1),
                                 cache_config=types.SimpleNamespace(block_size=T),
                                 kv_transfer_config=types.SimpleNamespace(kv_role="kv_both", kv_connector_extra_config=extra))


def caches(seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return {f"model.layers.{l}.self_attn.attn": torch.randn((2, NB, T, H, D), generator=g, device="cuda").to(torch.bfloat16)
            for l in range(L)}


def hashes(n, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, 16, size=32, dtype=np.uint8).astype("S1").tobytes().hex()[:32] for _ in range(n)]


def run_cycle(conn, kv, dump_reqs):
    conn.register_kv_caches(kv)
    conn.bind_connector_metadata(UCConnectorV1Metadata(dump_reqs))
    for name, layer in kv.items():
        conn.save_kv_layer(name, layer)
    done = conn.wait_for_save()
    conn.clear_connector_metadata()
    return done


@pytest.mark.parametrize("store_name", ["UcmDramStore", "UcmNfsStore"])
def test_dump_then_load_into_other_slots(tmp_path, store_name):
    cfg = {"storage_backends": str(tmp_path), "max_cache_size": 1 << 26}
    conn = UnifiedCacheConnectorV1(fake_config({"ucm_connector_name": store_name, "ucm_connector_config": cfg}), "worker", rank=0)
    kv = caches(1)
    hs = hashes(7, 2)
    src = [5, 0, 17, 9, 23, 2, 11]
    reqs = [ReqMeta("a", dump_blocks=list(zip(hs[:4], src[:4]))), ReqMeta("b", dump_blocks=list(zip(hs[4:], src[4:])))]
    assert conn.connector.create(hs) == [0] * len(hs)
    done = run_cycle(conn, kv, reqs)
    assert done == {"a": hs[:4], "b": hs[4:]}
    conn.connector.commit(hs, True)
    assert all(conn.connector.lookup(hs))
    # load: synchronous request and asynchronous request, into fresh caches at other block ids
    kv2 = {n: torch.zeros_like(t) for n, t in kv.items()}
    dst = [1, 22, 3, 14, 8, 19, 6]
    conn.register_kv_caches(kv2)
    conn.bind_connector_metadata(UCConnectorV1Metadata([ReqMeta("c", load_blocks=list(zip(hs[:4], dst[:4]))),
                                                        ReqMeta("d", load_blocks=list(zip(hs[4:], dst[4:])), load_async=True)]))
    conn.start_load_kv()
    for name in kv2:
        conn.wait_for_layer_load(name)
    finished = set()
    for _ in range(2000):
        finished |= conn.get_finished(set())[1]
        if "d" in finished:
            break
    assert finished == {"d"} and not conn.get_block_ids_with_load_errors()
    torch.cuda.synchronize()
    for name in kv:
        assert torch.equal(kv2[name][:, dst], kv[name][:, src])
        rest = sorted(set(range(NB)) - set(dst))
        assert not kv2[name][:, rest].any()
    assert N.device_error() == 0
    if hasattr(conn.connector, "close"):
        conn.connector.close()


def test_batched_dump_leaves_the_bytes_of_the_per_block_pattern(tmp_path):
    """Store A: this connector's one table per layer.  Store B: the reference's call pattern - one dump
    per block, layer and K/V with a tensor view and DataOffset (uc_connector.py:395-424).  Same files."""
    kv = caches(3)
    hs = hashes(5, 4)
    ids = [4, 13, 7, 20, 1]
    dirs = [tmp_path / "a", tmp_path / "b"]
    for d in dirs:
        d.mkdir()
    ca = UnifiedCacheConnectorV1(fake_config({"ucm_connector_name": "UcmNfsStore", "ucm_connector_config": {"storage_backends": str(dirs[0])}}), "worker")
    cb = UnifiedCacheConnectorV1(fake_config({"ucm_connector_name": "UcmNfsStore", "ucm_connector_config": {"storage_backends": str(dirs[1])}}), "worker")
    for c in (ca, cb):
        assert c.connector.create(hs) == [0] * len(hs)
    assert run_cycle(ca, kv, [ReqMeta("r", dump_blocks=list(zip(hs, ids)))]) == {"r": hs}
    tasks = []
    for name, layer in kv.items():
        tensors, offsets = cb.get_tensor_and_offset_layerwise(ids, layer, name)
        torch.cuda.current_stream().synchronize()
        for block_id, offset, tensor in zip(hs + hs, offsets, tensors):
            tasks.append(cb.connector.dump([block_id], [offset], [tensor]))
    assert all(cb.connector.wait(t) == 0 for t in tasks)
    for c in (ca, cb):
        c.connector.commit(hs, True)
    for h in hs:
        a = np.fromfile(ca.connector.path(h), dtype=np.uint8)
        b = np.fromfile(cb.connector.path(h), dtype=np.uint8)
        assert a.size == T * H * D * 2 * 2 * L
        np.testing.assert_array_equal(a, b)
    # and the stored block is [layer][K then V] of the cache bytes
    blob = np.fromfile(ca.connector.path(hs[2]), dtype=np.uint8)
    want = np.concatenate([kv[n][p, ids[2]].contiguous().view(torch.uint8).cpu().numpy().reshape(-1) for n in kv for p in (0, 1)])
    np.testing.assert_array_equal(blob, want)
    ca.connector.close(), cb.connector.close()
