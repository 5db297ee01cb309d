"""File-per-block store: on-disk layout and block life cycle against what the reference's own space
manager produced (tests/golden/nfs_layout.json, and the compiled reference itself when it is built),
plus host-memory dump/load through the worker threads.  No GPU needed."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from oracle import oracle
from ucmx import _native as N
from ucmx.store.factory import UcmConnectorFactory
from ucmx.store.nfsstore import UcmNfsStore

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "nfs_layout.json")))
IDS = [bytes.fromhex(h) for h in GOLD["ids"]]
need_ref = pytest.mark.skipif(not oracle.have_nfs_ref(), reason="the compiled reference space manager is not built")


def listing(root):
    out = []
    for r, ds, fs in os.walk(root):
        rel = os.path.relpath(r, root)
        for f in fs:
            out.append([os.path.join(rel, f), os.path.getsize(os.path.join(r, f))])
        if not ds and not fs:
            out.append([rel + "/", -1])
    return sorted(out)


def make_store(root, temp=False, role="worker", **kw):
    cfg = {"storage_backends": str(root), "kv_block_size": GOLD["block_size"], "role": role, "device": -1,
           "io_size": 4096, "temp_dump_dir_enable": temp}
    cfg.update(kw)
    return UcmNfsStore(cfg)


def replay(store, trace):
    got = []
    for op, hexid, _ in trace:
        bid = bytes.fromhex(hexid)
        if op == "new":
            got.append([op, hexid, store.create([bid])[0]])
        elif op == "lookup":
            got.append([op, hexid, int(store.lookup([bid])[0])])
        else:
            st = N.lib.ucmx_fstore_commit(store._h, bid, len(bid), 1 if op == "commit" else 0)
            got.append([op, hexid, st])
    return got


@pytest.mark.parametrize("mode", ["plain", "temp"])
def test_paths_and_life_cycle_match_recorded_reference(tmp_path, mode):
    gold = GOLD["layouts"][mode]
    store = make_store(tmp_path, temp=(mode == "temp"), role="scheduler")
    for bid, (act, dat) in zip(IDS, gold["paths"]):
        assert os.path.relpath(store.path(bid, True), tmp_path) == act
        assert os.path.relpath(store.path(bid, False), tmp_path) == dat
    assert replay(store, gold["trace"]) == gold["trace"]
    assert listing(tmp_path) == [list(x) for x in gold["listing"]]
    store.close()


def test_backend_choice_matches_recorded_reference(tmp_path):
    roots = [tmp_path / n for n in ("b0", "b1", "b2")]
    for r in roots:
        (r / "data").mkdir(parents=True)
    store = make_store(":".join(str(r) for r in roots), role="scheduler")
    got = [int(os.path.relpath(store.path(b, False), tmp_path)[1]) for b in IDS]
    assert got == GOLD["backend_of"]
    store.close()


def test_setup_errors(tmp_path):
    with pytest.raises(RuntimeError, match="errcode: -50002"):
        make_store(tmp_path / "missing" / "deeper")                      # parent directory does not exist
    (tmp_path / "a").mkdir()
    with pytest.raises(RuntimeError, match="errcode: -50000"):
        make_store(f"{tmp_path / 'a'}:{tmp_path / 'no_such_backend'}")   # secondary backends must exist already
    with pytest.raises(RuntimeError, match="errcode: -50000"):
        UcmNfsStore({"storage_backends": str(tmp_path), "kv_block_size": 0, "role": "scheduler"})
    store = make_store(tmp_path, role="scheduler")
    with pytest.raises(ValueError):
        store.create(["short-id"])
    # a store without workers refuses transfers and wait() reports the invalid task
    t = store.dump_from_host([IDS[0]], [0], [0], [16])
    assert t.task_id == 0 and store.wait(t) == N.ENOOBJ
    store.close()


@need_ref
@pytest.mark.parametrize("temp", [False, True])
def test_live_reference_agrees_on_random_ids(tmp_path, temp):
    rng = np.random.default_rng(7)
    ours_root, ref_root = tmp_path / "ours", tmp_path / "ref"
    ours_root.mkdir(), ref_root.mkdir()
    store = make_store(ours_root, temp=temp, role="scheduler")
    ref = oracle.RefSpaceManager(str(ref_root), GOLD["block_size"], temp)
    ids = [rng.integers(0, 256, size=int(n), dtype=np.uint8).tobytes() for n in rng.integers(16, 40, size=64)]
    ids = [i.replace(b"\0", b"\1") for i in ids]    # ids travel as C strings on the Python side of the reference
    for bid in ids:
        for act in (True, False):
            assert os.path.relpath(store.path(bid, act), ours_root) == os.path.relpath(ref.path(bid, act), ref_root)
    for step in range(400):
        bid = ids[int(rng.integers(0, len(ids)))]
        op = int(rng.integers(0, 4))
        if op == 0:
            assert store.create([bid])[0] == ref.new_block(bid), step
        elif op == 1:
            assert store.lookup([bid])[0] == ref.lookup(bid), step
        else:
            ok = op == 2
            assert N.lib.ucmx_fstore_commit(store._h, bid, len(bid), int(ok)) == ref.commit(bid, ok), step
    assert listing(ours_root) == listing(ref_root)
    store.close()


def _host_round_trip(store, ids, n_slices, slice_bytes, rng):
    data = {b: rng.integers(0, 256, size=(n_slices, slice_bytes), dtype=np.uint8) for b in ids}
    assert store.create(ids) == [0] * len(ids)
    bl, off, adr, sz = [], [], [], []
    for b in ids:
        for s in range(n_slices):
            bl.append(b), off.append(s * slice_bytes), adr.append(data[b][s].ctypes.data), sz.append(slice_bytes)
    task = store.dump_from_host(bl, off, adr, sz)
    assert task.task_id > 0
    assert store.wait(task) == 0
    store.commit(ids, True)
    assert store.lookup(ids) == [True] * len(ids)
    back = {b: np.zeros_like(data[b]) for b in ids}
    adr = [back[b][s].ctypes.data for b in ids for s in range(n_slices)]
    task = store.load_to_host(bl, off, adr, sz)
    st, _ = store.check(task)
    assert st == 0
    assert store.wait(task) == 0
    assert store.check(task)[0] == N.ENOOBJ      # a waited task is forgotten
    for b in ids:
        np.testing.assert_array_equal(back[b], data[b])
    return data


@pytest.mark.parametrize("slice_bytes", [4096, 1000])
def test_host_dump_load_round_trip(tmp_path, slice_bytes):
    rng = np.random.default_rng(11)
    store = make_store(tmp_path, stream_number=3)
    _host_round_trip(store, IDS[1:8], GOLD["block_size"] // 4096, slice_bytes, rng)
    store.close()


@need_ref
def test_files_interchange_with_reference(tmp_path):
    rng = np.random.default_rng(13)
    store = make_store(tmp_path, stream_number=2)
    ids = IDS[4:8]
    data = _host_round_trip(store, ids, 4, 4096, rng)
    ref = oracle.RefSpaceManager(str(tmp_path), GOLD["block_size"], False)
    # the reference reads what we wrote ...
    for b in ids:
        assert ref.lookup(b)
        out = np.zeros((4, 4096), np.uint8)
        assert ref.read(ref.path(b, False), 0, out) == 0
        np.testing.assert_array_equal(out, data[b])
    # ... and we read what the reference writes
    b = IDS[9]
    payload = rng.integers(0, 256, size=GOLD["block_size"], dtype=np.uint8)
    assert ref.new_block(b) == 0
    assert ref.write(ref.path(b, True), 0, payload) == 0
    assert ref.commit(b, True) == 0
    got = np.zeros(8192, np.uint8)
    task = store.load_to_host([b], [12288], [got.ctypes.data], [8192])
    assert store.wait(task) == 0
    np.testing.assert_array_equal(got, payload[12288:12288 + 8192])
    store.close()


def test_failed_slice_fails_the_task(tmp_path):
    store = make_store(tmp_path, stream_number=2)
    buf = np.zeros(4096, np.uint8)
    # loading a block that was never committed: the task finishes, with an error
    task = store.load_to_host([IDS[0], IDS[1]], [0, 0], [buf.ctypes.data] * 2, [4096] * 2)
    assert store.wait(task) == N.ERROR
    # reading past the end of a block file is a short read, hence a failure, as in the reference
    assert store.create([IDS[3]]) == [0]
    store.commit([IDS[3]], True)
    task = store.load_to_host([IDS[3]], [GOLD["block_size"] - 1024], [buf.ctypes.data], [4096])
    assert store.wait(task) == N.ERROR
    assert store.wait(task) == N.ENOOBJ
    store.close()


def test_factory_builds_the_store(tmp_path):
    s = UcmConnectorFactory.create_connector("UcmNfsStore", {"storage_backends": str(tmp_path), "kv_block_size": 4096,
                                                             "role": "scheduler"})
    assert isinstance(s, UcmNfsStore) and s.cc_store() != 0
    s.close()
