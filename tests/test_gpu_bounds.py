"""Ids that point outside the table or cache they index are skipped and reported (device error code 3), never turned
into an address; bad arguments that are visible on the host are refused before anything is launched.  Nothing here
makes the GPU touch memory it does not own."""
import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


def dev_bf16(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(DEV).view(torch.bfloat16)


@pytest.mark.parametrize("Hkv,D,n_rep", [(8, 128, 1), (1, 128, 1), (2, 64, 2), (8, 128, 2), (4, 128, 4), (8, 128, 4)])
# (copy-engine rows, narrow rows, general kernel, copy-engine rows with two and four representatives, whole row in flight)
def test_score_dot_skips_slots_beyond_the_table(oracle, Hkv, D, n_rep):
    from ucmx import _native, ops
    rng = np.random.default_rng(201)
    n_slots = 300
    reps16 = H.randn_bf16(rng, (n_slots, Hkv, n_rep, D), 0.09)
    off = H.ragged_offsets([120, 80])
    slots = rng.integers(0, n_slots, 200).astype(np.int32)
    bad = [3, 77, 150, 199]
    slots[bad] = [n_slots, n_slots + 5, 2_000_000_000, n_slots]
    q = H.bf16_to_f32(H.randn_bf16(rng, (2, Hkv * D)))
    _native.device_error()
    got = ops.score_dot(dev_bf16(reps16), dev_i32(off), torch.from_numpy(q).to(DEV), total=200, slot_ids=dev_i32(slots),
                        n_kv_heads=Hkv, head_dim=D, n_rep=n_rep).cpu().numpy()
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert np.all(np.isneginf(got[bad]))
    ok = np.setdiff1d(np.arange(200), bad)
    safe = slots.copy()
    safe[bad] = 0
    if n_rep == 1:
        ref = oracle.score_dot_esa(H.bf16_to_f32(reps16).reshape(n_slots, -1), off, safe, q)
    else:
        ref = oracle.score_dot_gsa(H.bf16_to_f32(reps16), Hkv, n_rep, D, off, safe, q)
    np.testing.assert_allclose(got[ok], ref[ok], rtol=1e-3, atol=1e-3 * float(np.abs(ref).std()))


def test_score_dot_heads_and_fused_query_skip_bad_slots():
    from ucmx import _native, ops
    rng = np.random.default_rng(202)
    reps = dev_bf16(H.randn_bf16(rng, (64, 8, 1, 128), 0.09))
    q = dev_bf16(H.randn_bf16(rng, (1, 32, 128)))
    slots = np.arange(50, dtype=np.int32)
    slots[7] = 64
    _native.device_error()
    a = ops.score_dot_heads(reps, dev_i32([0, 50]), q, total=50, slot_ids=dev_i32(slots)).cpu().numpy()
    b = ops.score_dot_query(reps, dev_i32([0, 50]), q, total=50, slot_ids=dev_i32(slots), n_kv_heads=8).cpu().numpy()
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert np.isneginf(a[7]) and np.isneginf(b[7]) and np.isfinite(np.delete(a, 7)).all() and np.isfinite(np.delete(b, 7)).all()


def test_gather_scatter_and_move_skip_blocks_beyond_the_cache():
    from ucmx import _native, ops
    g = torch.Generator(device=DEV).manual_seed(203)
    k = torch.randint(0, 255, (40, 4096), generator=g, device=DEV, dtype=torch.uint8)
    v = torch.randint(0, 255, (40, 4096), generator=g, device=DEV, dtype=torch.uint8)
    ids = dev_i32([5, 40, 39, -1, 1000, 0])
    staging = torch.full((6, 2, 4096), 7, dtype=torch.uint8, device=DEV)
    _native.device_error()
    ops.gather_blocks([k, v], ids, staging)
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    for i, b in enumerate([5, None, 39, None, None, 0]):
        if b is None:
            assert bool((staging[i] == 7).all())                      # untouched
        else:
            assert torch.equal(staging[i, 0], k[b]) and torch.equal(staging[i, 1], v[b])
    k2, v2 = k.clone(), v.clone()
    ops.scatter_blocks([k2, v2], dev_i32([40, 3]), staging[:2].contiguous())
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert torch.equal(k2[3], staging[1, 0]) and torch.equal(torch.cat([k2[:3], k2[4:]]), torch.cat([k[:3], k[4:]]))
    # block-to-block moves: pairs with an id out of range on either side are left alone
    dk, dv = torch.zeros((10, 4096), dtype=torch.uint8, device=DEV), torch.zeros((10, 4096), dtype=torch.uint8, device=DEV)
    ops.move_blocks([k, v], dev_i32([1, 2, 40, 3, -1]), [dk, dv], dev_i32([9, 0, 1, 10, 2]))
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert torch.equal(dk[9], k[1]) and torch.equal(dv[0], v[2]) and not bool(dk[1].any()) and not bool(dk[2].any())


def test_move_list_length_is_read_on_the_device():
    from ucmx import _native, ops
    g = torch.Generator(device=DEV).manual_seed(204)
    src = [torch.randint(0, 255, (64, 8192), generator=g, device=DEV, dtype=torch.uint8) for _ in range(2)]
    dst = [torch.zeros((32, 8192), dtype=torch.uint8, device=DEV) for _ in range(2)]
    moves = ops.MoveList(20, torch.device(DEV))
    moves.src[:5] = dev_i32([3, 60, 7, 8, 9])
    moves.dst[:5] = dev_i32([0, 31, 2, 3, 4])
    moves.src[5:] = 1                                   # stale entries behind the list's end must not move
    moves.dst[5:] = 20
    for n in (3, 5, 0):
        for d in dst:
            d.zero_()
        moves.count[0] = n
        ops.move_blocks(src, moves, dst)
        torch.cuda.synchronize()
        assert moves.count.cpu().tolist() == [0, 0]     # consumed
        for i in range(5):
            s, d = int(moves.src[i]), int(moves.dst[i])
            for p in range(2):
                assert torch.equal(dst[p][d], src[p][s]) if i < n else not bool(dst[p][d].any())
        assert not bool(dst[0][20].any())
    assert _native.device_error() == 0


def test_remap_refuses_a_request_with_more_slots_than_declared():
    from ucmx import _native, ops
    n = 12
    slot_logical = torch.full((n,), -1, dtype=torch.int32, device=DEV)
    slot_free = torch.ones((n,), dtype=torch.uint8, device=DEV)
    slot_phys = torch.arange(n, dtype=torch.int32, device=DEV)
    off = dev_i32([0, 4, 12])                          # the second request owns 8 slots, 6 are declared
    sel, sel_off = dev_i32([0, 1, 2, 0, 1, 2, 3]), dev_i32([0, 3, 7])
    _native.device_error()
    table, ll, lp, cnt = ops.remap_resident(slot_logical, slot_free, slot_phys, off, sel, sel_off, max_logical=16, max_slots=6)
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert cnt.cpu().tolist() == [3, 0]
    assert table.cpu().tolist()[:3] == [0, 1, 2] and table.cpu().tolist()[3:] == [-1] * 4
    assert slot_logical.cpu().tolist()[4:] == [-1] * 8 and bool(slot_free[4:].all())     # its state was not touched


def test_retrieval_submit_refuses_indexes_outside_the_table():
    from ucmx import _native
    from ucmx.retrieval import RetrievalWorkerBackend
    rng = np.random.default_rng(205)
    be = RetrievalWorkerBackend(rng.standard_normal((50, 64), dtype=np.float32))
    q = rng.standard_normal((1, 64), dtype=np.float32)
    for bad in (50, 1 << 30, -2):
        idx = np.array([[0, 1, bad, -1]], np.int32)
        with pytest.raises(_native.UcmxError) as e:
            be.submit(q, 2, idx)
        assert e.value.status == _native.EPARAM and "outside the table" in str(e.value)
    rid = be.submit(q, 2, np.array([[0, 1, 49, -1]], np.int32))       # -1 pads, 49 is the last row
    be.wait(rid)
    assert be.get_result(rid)["indices"].shape == (1, 2)
    be.close()
    assert _native.device_error() == 0


def test_pooling_hashing_and_hamming_drop_ids_beyond_their_tables(oracle):
    """Block ids beyond the cache, output rows beyond the table, code-table slots beyond the table: dropped, reported."""
    from ucmx import _native, ops
    rng = np.random.default_rng(206)
    k16 = H.randn_bf16(rng, (6, 16, 2, 128))
    k = dev_bf16(k16)
    table = torch.zeros((4, 2, 1, 128), dtype=torch.bfloat16, device=DEV)
    _native.device_error()
    ops.pool_blocks(k, dev_i32([1, 6, 2, 5]), out_slots=dev_i32([0, 1, 4, 3]), out_bf16=table)   # id 6 and row 4 do not exist
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    want = H.f32_to_bf16(oracle.pool_blocks(k16, np.asarray([1, 5], np.int32), 0, True))
    got = table.view(torch.int16).cpu().numpy().view(np.uint16).reshape(4, -1)
    assert np.array_equal(got[[0, 3]], want) and not got[[1, 2]].any()
    # a larger batch takes the streaming kernel
    ids = np.arange(600, dtype=np.int32) % 6
    ids[[17, 400]] = [6, 99]
    big = torch.zeros((600, 2, 1, 128), dtype=torch.bfloat16, device=DEV)
    ops.pool_blocks(k, dev_i32(ids), out_bf16=big)
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    gotb = big.view(torch.int16).cpu().numpy().view(np.uint16).reshape(600, -1)
    ref = H.f32_to_bf16(oracle.pool_blocks(k16, np.arange(6, dtype=np.int32), 0, True))
    assert not gotb[[17, 400]].any() and np.array_equal(gotb[5], ref[5]) and np.array_equal(gotb[599], ref[599 % 6])
    # hash codes of blocks: tensor-core shape (128 channels, 128 bits)
    w = dev_bf16(H.randn_bf16(rng, (128, 128), 2.0))
    codes = torch.zeros((3, 2, 16, 16), dtype=torch.uint8, device=DEV)
    ops.hash_encode_blocks(k, dev_i32([0, 7, 3]), w, out=codes)
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert not bool(codes[1].any()) and bool(codes[0].any()) and bool(codes[2].any())
    # Hamming scores: a slot beyond the code table
    ctab = torch.randint(0, 255, (5, 2, 16, 16), dtype=torch.uint8, device=DEV)
    qc = torch.randint(0, 255, (1, 2, 16), dtype=torch.uint8, device=DEV)
    s = ops.score_hamming(ctab, dev_i32([0, 4]), qc, total=4, slot_ids=dev_i32([0, 5, 4, -1])).cpu().numpy()
    torch.cuda.synchronize()
    assert _native.device_error() == 3
    assert s[1] == np.iinfo(np.int32).min and s[3] == np.iinfo(np.int32).min and s[0] > np.iinfo(np.int32).min
