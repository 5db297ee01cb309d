"""File-per-block store, device leg: KV slices dumped from HBM to block files and loaded back into
other slots must come back bit-identical, for every staging shape (whole groups in one launch, slices
longer than a slot, sizes the batched kernel cannot take)."""
import numpy as np
import pytest
import torch

from ucmx import _native as N
from ucmx.store.dramstore import store_offset
from ucmx.store.nfsstore import UcmNfsStore

pytestmark = pytest.mark.gpu


def _ids(n, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(1, 256, size=32, dtype=np.uint8).tobytes() for _ in range(n)]


def _store(tmp_path, block_bytes, io_size, **kw):
    cfg = {"storage_backends": str(tmp_path), "kv_block_size": block_bytes, "role": "worker", "device": 0,
           "io_size": io_size}
    cfg.update(kw)
    return UcmNfsStore(cfg)


@pytest.mark.parametrize("io_size,slots,workers", [(4096, 16, 4), (4096, 2, 1), (1024, 6, 3)])
def test_kv_slices_round_trip_through_block_files(tmp_path, io_size, slots, workers):
    L, T, H, D, nb, n = 4, 16, 2, 64, 40, 12
    g = torch.Generator(device="cuda").manual_seed(5)
    k = [torch.randn((nb, T, H, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(L)]
    v = [torch.randn((nb, T, H, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(L)]
    slice_bytes = T * H * D * 2
    block_bytes = slice_bytes * 2 * L
    store = _store(tmp_path, block_bytes, io_size, buffer_number=slots, stream_number=workers)
    ids = _ids(n, 1)
    src = torch.randperm(nb)[:n].tolist()
    assert store.create(ids) == [0] * n
    bl, off, ten = [], [], []
    for b, s in zip(ids, src):
        for l in range(L):
            for is_v, cache in ((False, k), (True, v)):
                bl.append(b), off.append(store_offset((T, H, D), 0, 1, 2, l, is_v)), ten.append(cache[l][s])
    task = store.dump(bl, off, ten)
    assert store.wait(task) == 0
    store.commit(ids, True)
    assert all(store.lookup(ids))
    # into other slots of fresh caches
    k2 = [torch.zeros_like(x) for x in k]
    v2 = [torch.zeros_like(x) for x in v]
    dst = torch.randperm(nb)[:n].tolist()
    ten = []
    for b, s in zip(ids, dst):
        for l in range(L):
            ten.append(k2[l][s]), ten.append(v2[l][s])
    task = store.load(bl, off, ten)
    assert store.wait(task) == 0
    torch.cuda.synchronize()
    for l in range(L):
        assert torch.equal(k2[l][dst], k[l][src]) and torch.equal(v2[l][dst], v[l][src])
        untouched = sorted(set(range(nb)) - set(dst))
        assert not k2[l][untouched].any() and not v2[l][untouched].any()
    assert N.device_error() == 0
    store.close()


@pytest.mark.parametrize("nbytes", [1000, 40 * 1024 + 16, 6])
def test_odd_slice_sizes(tmp_path, nbytes):
    store = _store(tmp_path, 1 << 20, 16384, buffer_number=4, stream_number=2)
    ids = _ids(5, 2)
    g = torch.Generator(device="cuda").manual_seed(9)
    src = [torch.randint(0, 256, (nbytes,), generator=g, device="cuda", dtype=torch.uint8) for _ in ids]
    offs = [4096 * (i + 1) + (3 if nbytes == 6 else 0) for i in range(len(ids))]
    assert store.create(ids) == [0] * len(ids)
    assert store.wait(store.dump(ids, offs, src)) == 0
    store.commit(ids, True)
    dst = [torch.zeros_like(s) for s in src]
    assert store.wait(store.load(ids, offs, dst)) == 0
    torch.cuda.synchronize()
    for a, b in zip(src, dst):
        assert torch.equal(a, b)
    # and the bytes on disk are the bytes of the tensors
    raw = np.fromfile(store.path(ids[2]), dtype=np.uint8)
    assert raw.size == 1 << 20
    np.testing.assert_array_equal(raw[offs[2]:offs[2] + nbytes], src[2].cpu().numpy())
    store.close()


def test_missing_block_fails_the_device_load(tmp_path):
    store = _store(tmp_path, 65536, 4096)
    dst = [torch.zeros(4096, dtype=torch.uint8, device="cuda")]
    assert store.wait(store.load(_ids(1, 3), [0], dst)) == N.ERROR
    store.close()
