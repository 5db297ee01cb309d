"""GSAPrefetchTables (device-side block tables of GSA) against the CPU checker's restatement of the reference's
prefetch engine round, request by request and layer by layer."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_block_tables_follow_the_prefetch_engine(oracle):
    from ucmx import _native
    from ucmx.sparse.gsa_prefetch import GSAPrefetchTables
    rng = np.random.default_rng(501)
    L, max_bs, max_blocks, max_slots, T = 3, 6, 300, 24, 16
    tables = GSAPrefetchTables(L, max_bs, max_blocks, max_slots, T, torch.device(DEV))
    reqs = {"a": dict(n=210, hbm=sorted(rng.choice(5000, 20, replace=False).tolist()), k=17, seq=210 * T - 5),
            "b": dict(n=90, hbm=sorted(rng.choice(5000, 24, replace=False).tolist()), k=24, seq=89 * T + 1),
            "c": dict(n=35, hbm=sorted(rng.choice(5000, 9, replace=False).tolist()), k=8, seq=35 * T)}
    # host-side mirror of the state, one copy per (request, layer)
    mirror = {}
    for name, r in reqs.items():
        row = tables.add_request(name, r["hbm"])
        assert tables.rows[name] == row
        for l in range(L):
            mirror[(name, l)] = (np.full(len(r["hbm"]), -1, np.int32), np.ones(len(r["hbm"]), np.uint8), np.asarray(r["hbm"], np.int32))
    _native.device_error()
    for rnd in range(5):
        batch = ["a", "b", "c"] if rnd != 2 else ["c", "a"]            # one round without request b: its state must not move
        width = max(reqs[n]["k"] for n in batch)
        topk = np.full((L, len(batch), width), -1, np.int32)
        for l in range(L):
            for i, n in enumerate(batch):
                topk[l, i, :reqs[n]["k"]] = np.sort(rng.choice(reqs[n]["n"], reqs[n]["k"], replace=False))
        ll, lp, lc = tables.run_prefetch(batch, torch.from_numpy(topk).to(DEV), [reqs[n]["k"] for n in batch],
                                         [reqs[n]["seq"] for n in batch])
        mi = tables.model_input_del(batch)
        torch.cuda.synchronize()
        assert _native.device_error() == 0
        for l in range(L):
            bt, sl, bl = mi["block_tables_mp"][l].cpu().numpy(), mi["gsa_seq_len"][l].cpu().numpy(), mi["block_table_len"][l].cpu().numpy()
            for i, n in enumerate(batch):
                k = reqs[n]["k"]
                res, fr, phys = mirror[(n, l)]
                res2, fr2, table, want_ll, want_lp = oracle.remap_resident(res, fr, phys, topk[l, i, :k])
                mirror[(n, l)] = (res2, fr2, phys)
                row = tables.rows[n]
                assert bl[i] == k and np.array_equal(bt[i, :k], table)
                nl = int(lc[l, row])
                assert nl == len(want_ll)
                assert np.array_equal(ll[l, row, :nl].cpu().numpy(), want_ll) and np.array_equal(lp[l, row, :nl].cpu().numpy(), want_lp)
                ns = len(phys)
                assert np.array_equal(tables.slot_logical[l, row, :ns].cpu().numpy(), res2)
                assert np.array_equal(tables.slot_free[l, row, :ns].cpu().numpy(), fr2)
                tail = reqs[n]["seq"] - ((reqs[n]["seq"] - 1) // T) * T
                assert sl[i] == (k - 1) * T + tail
    tables.del_request("b")
    assert "b" not in tables.rows and int(tables.block_table_len[:, 1].sum()) == 0
    assert tables.add_request("d", [7, 3, 5], resident=[40, -1, 2]) == 1            # the freed row is reused; blocks sorted by id
    assert tables.slot_phys[0, 1, :3].cpu().tolist() == [3, 5, 7] and tables.slot_logical[0, 1, :3].cpu().tolist() == [-1, 2, 40]
    assert tables.slot_free[0, 1, :3].cpu().tolist() == [1, 0, 0]
