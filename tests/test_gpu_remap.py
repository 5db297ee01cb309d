"""Resident-set remap on the device against the CPU restatement of the reference's prefetch engine
(GetHitAndMissBlock / RunPrefetchH2D / LoadKVToHBM), over several rounds with carried state."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dt=np.int32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=dt)).to(DEV)


def test_remap_rounds_match_checker(oracle):
    from ucmx import ops
    rng = np.random.default_rng(91)
    n_logical = [300, 64, 1000, 17]               # blocks of each request's context
    n_slots = [40, 64, 90, 5]                     # HBM blocks each request owns
    ks = [30, 70, 80, 9]                          # selected per round (may exceed what fits)
    slot_off = H.ragged_offsets(n_slots)
    phys, logical, free = [], [], []
    next_phys = 0
    for r, ns in enumerate(n_slots):
        ids = np.sort(rng.choice(np.arange(next_phys, next_phys + 3 * ns), ns, replace=False)).astype(np.int32)
        next_phys += 3 * ns
        phys.append(ids)
        start = rng.choice(n_logical[r], min(ns, n_logical[r]) // 2, replace=False).astype(np.int32)
        lg = np.full(ns, -1, np.int32)
        lg[rng.permutation(ns)[: len(start)]] = start        # half of the slots hold something
        logical.append(lg)
        free.append((lg < 0).astype(np.uint8))               # the empty ones are on the free list
    d_logical, d_free = dev(np.concatenate(logical)), dev(np.concatenate(free), np.uint8)
    d_phys, d_slot_off = dev(np.concatenate(phys)), dev(slot_off)
    sel_off = H.ragged_offsets(ks)
    for rnd in range(5):
        sels = [np.sort(rng.choice(n_logical[r], min(ks[r], n_logical[r]), replace=False)).astype(np.int32) for r in range(4)]
        flat = np.full(int(sel_off[-1]), -1, np.int32)
        counts = np.zeros(4, np.int32)
        for r in range(4):
            flat[sel_off[r]: sel_off[r] + len(sels[r])] = sels[r]
            counts[r] = len(sels[r])
        table, ll, lp, lc = ops.remap_resident(d_logical, d_free, d_phys, d_slot_off, dev(flat), dev(sel_off),
                                               max_logical=1000, max_slots=90, sel_counts=dev(counts))
        table, ll, lp, lc = table.cpu().numpy(), ll.cpu().numpy(), lp.cpu().numpy(), lc.cpu().numpy()
        new_logical, new_free = d_logical.cpu().numpy(), d_free.cpu().numpy()
        for r in range(4):
            wl, wf, wt, wll, wlp = oracle.remap_resident(logical[r], free[r], phys[r], sels[r])
            a, b = sel_off[r], sel_off[r] + len(sels[r])
            assert np.array_equal(table[a:b], wt), (rnd, r)
            assert lc[r] == len(wll)
            assert np.array_equal(ll[a:a + lc[r]], wll) and np.array_equal(lp[a:a + lc[r]], wlp)
            assert np.array_equal(new_logical[slot_off[r]:slot_off[r + 1]], wl)
            assert np.array_equal(new_free[slot_off[r]:slot_off[r + 1]], wf)
            # invariants: every served block is resident exactly once
            served = wt[wt >= 0]
            assert len(set(served.tolist())) == len(served)
            logical[r], free[r] = wl, wf
    from ucmx import _native
    assert _native.device_error() == 0


def test_remap_feeds_the_block_transfer(oracle):
    """top-k (ascending) -> remap -> scatter of the loaded blocks: the selected ids never leave the device."""
    from ucmx import ops
    rng = np.random.default_rng(92)
    n_blocks, slice_elems = 200, 1024
    store = rng.integers(0, 2**16, (n_blocks, slice_elems), dtype=np.uint16)      # every logical block, "in the store"
    hbm = np.zeros((64, slice_elems), np.uint16)
    slot_phys = np.sort(rng.choice(64, 24, replace=False)).astype(np.int32)
    d_logical, d_free = dev(np.full(24, -1)), dev(np.ones(24), np.uint8)
    d_hbm = torch.from_numpy(hbm.view(np.int16)).to(DEV)
    d_store = torch.from_numpy(store.view(np.int16)).to(DEV)
    scores = torch.from_numpy(rng.standard_normal(n_blocks).astype(np.float32)).to(DEV)
    off = dev([0, n_blocks])
    sel, _, cnt = ops.topk_ragged(scores, off, dev([20]), out_stride=20, order=ops.ORDER_INDEX_ASC, want_scores=False)
    table, ll, lp, lc = ops.remap_resident(d_logical, d_free, dev(slot_phys), dev([0, 24]), sel.view(-1), dev([0, 20]),
                                           max_logical=n_blocks, max_slots=24, sel_counts=cnt)
    n = int(lc.item())
    assert n == 20
    # gather the blocks to load from the "store" pool, scatter them into their HBM slots: two launches, ids on device
    staging = torch.empty(20 * slice_elems * 2, dtype=torch.uint8, device=DEV)
    ops.gather_blocks([d_store], ll, staging)
    ops.scatter_blocks([d_hbm], lp, staging)
    torch.cuda.synchronize()
    got = d_hbm.cpu().numpy().view(np.uint16)
    t, s = table.cpu().numpy(), sel.cpu().numpy().reshape(-1)
    for j in range(20):
        assert np.array_equal(got[t[j]], store[s[j]])


@pytest.mark.parametrize("name", list(H.REMAP_SCENARIOS))
def test_remap_replays_recorded_prefetch_engine(name):
    """The device kernel against recorded runs of the reference's GSAPrefetchEngineC itself
    (tests/golden/remap_rounds.json): every layer of a scenario is one entry of a single ragged launch."""
    import json
    import os

    from ucmx import ops
    with open(os.path.join(os.path.dirname(__file__), "golden", "remap_rounds.json")) as f:
        recorded = {c["name"]: c["rounds"] for c in json.load(f)}[name]
    sc = H.remap_scenario(name)
    L, bt = sc["n_layers"], sc["block_table"]
    order = sorted(sc["owned_idx"], key=lambda i: bt[i])
    phys = np.asarray([bt[i] for i in order], np.int32)
    ns = len(order)
    d_logical = dev(np.tile(np.asarray(order, np.int32), L))
    d_free = dev(np.tile(np.asarray([1 if i in sc["free_idx"] else 0 for i in order], np.uint8), L), np.uint8)
    d_phys, d_slot_off = dev(np.tile(phys, L)), dev(np.arange(L + 1) * ns)
    for sel, want in zip(sc["rounds"], recorded):
        k = sel.shape[1]
        table, ll, lp, lc = ops.remap_resident(d_logical, d_free, d_phys, d_slot_off, dev(sel.reshape(-1)), dev(np.arange(L + 1) * k),
                                               max_logical=len(bt), max_slots=ns)
        table, ll, lp, lc = table.cpu().numpy(), ll.cpu().numpy(), lp.cpu().numpy(), lc.cpu().numpy()
        logical, free = d_logical.cpu().numpy().reshape(L, ns), d_free.cpu().numpy().reshape(L, ns)
        for l in range(L):
            pairs = sorted((int(s), int(t)) for s, t in zip(sel[l], table[l * k:(l + 1) * k]) if t >= 0)
            assert [t for _, t in pairs] == want["table"][l]
            assert lp[l * k: l * k + lc[l]].tolist() == want["load_blocks"][l]
            assert ll[l * k: l * k + lc[l]].tolist() == want["miss_idx"][l][: lc[l]]
            assert [int(p) for p, f in zip(phys, free[l]) if f] == want["free"][l]
            assert {str(int(p)): int(x) for p, x in zip(phys, logical[l])} == want["blocks_map"][l]


def test_packed_move_list_equals_the_per_request_load_lists():
    """With a move list, a round also leaves ONE list (block to read in the pool -> HBM block) for the whole batch:
    the same loads as the per-request lists hold, each mapped through the request's row of the block table."""
    from ucmx import ops
    rng = np.random.default_rng(303)
    n_req = 9
    n_blocks = rng.integers(30, 200, n_req)
    ks = np.maximum(4, n_blocks // 6).astype(np.int32)
    boff = np.concatenate([[0], np.cumsum(n_blocks)]).astype(np.int32)
    koff = np.concatenate([[0], np.cumsum(ks)]).astype(np.int32)
    block_table = rng.permutation(int(boff[-1])).astype(np.int32)         # pool block of every logical block
    total_k = int(koff[-1])
    d_logical = dev(np.full(total_k, -1, np.int32))
    d_free = dev(np.ones(total_k, np.uint8), np.uint8)
    d_phys = dev(np.arange(total_k, dtype=np.int32))
    moves = ops.MoveList(total_k, torch.device(DEV))
    seen_moves = 0
    for rnd in range(4):
        sel = np.concatenate([np.sort(rng.choice(n_blocks[r], ks[r], replace=False)) for r in range(n_req)]).astype(np.int32)
        table, ll, lp, lc = ops.remap_resident(d_logical, d_free, d_phys, dev(koff), dev(sel), dev(koff),
                                               max_logical=int(n_blocks.max()), max_slots=int(ks.max()),
                                               src_map=dev(block_table), src_map_offsets=dev(boff), moves=moves)
        torch.cuda.synchronize()
        n = int(moves.count[0])
        ll, lp, lc = ll.cpu().numpy(), lp.cpu().numpy(), lc.cpu().numpy()
        assert n == int(lc.sum()) and int(moves.count[1]) == 0
        want = set()
        for r in range(n_req):
            for j in range(lc[r]):
                want.add((int(block_table[boff[r] + ll[koff[r] + j]]), int(lp[koff[r] + j])))
            assert (ll[koff[r] + lc[r]: koff[r + 1]] == -1).all() and (lp[koff[r] + lc[r]: koff[r + 1]] == -1).all()
        got = set(zip(moves.src[:n].cpu().tolist(), moves.dst[:n].cpu().tolist()))
        assert got == want and len(got) == n
        seen_moves += n
        moves.count.zero_()                                    # (move_blocks would do this)
        if rnd == 0:
            assert n == total_k                                # nothing was resident: every selected block is a load
    assert seen_moves < 4 * total_k                            # later rounds hit resident blocks
