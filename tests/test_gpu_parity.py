"""Parity of the CUDA path against the CPU checker, called through the C ABI (ucmx.ops -> libucmx.so).

Bit-exact for integer, byte and index work and for fp32 results whose operation order the kernel
shares with the checker (pooling, query means, hash codes); scores, whose summation order differs
(warp tree vs left-to-right), to 1e-3 relative of the score scale as the target states.
"""
import os

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))
DEV = "cuda:0"


def dev_bf16(u16):
    return torch.from_numpy(np.ascontiguousarray(u16).view(np.int16)).to(DEV).view(torch.bfloat16)


def host_bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def dev_i32(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32)).to(DEV)


@pytest.fixture(scope="module")
def ops():
    from ucmx import ops
    return ops


# --------------------------------------------------------------------------------- stage 1: pool

@pytest.mark.parametrize("mode,code", [("mean", 0), ("max", 1), ("min", 2), ("sum", 3)])
def test_pool_modes_bit_exact(ops, oracle, mode, code):
    k, ids = H.case_pool()
    kd = dev_bf16(k)
    f32 = torch.empty((len(ids), 1024), dtype=torch.float32, device=DEV)
    b16 = ops.pool_blocks(kd, dev_i32(ids), mode=mode, out_f32=f32,
                          out_bf16=torch.empty((len(ids), 8, 1, 128), dtype=torch.bfloat16, device=DEV))
    want = oracle.pool_blocks(k, ids, code, True)
    assert np.array_equal(f32.cpu().numpy(), want)
    assert np.array_equal(host_bits(b16).reshape(len(ids), 1024), H.f32_to_bf16(want))
    # unrounded fp32 (the GSA native representative)
    f32u = torch.empty_like(f32)
    ops.pool_blocks(kd, dev_i32(ids), mode=mode, out_f32=f32u, round_bf16=False)
    assert np.array_equal(f32u.cpu().numpy(), oracle.pool_blocks(k, ids, code, False))


def test_pool_matches_reference_vectors(ops):
    k, ids = H.case_pool()
    out = ops.pool_blocks(dev_bf16(k), dev_i32(ids))
    d = H.bf16_ulp_distance(host_bits(out).reshape(9, 8, 128), G["pool_mean"])
    assert d.max() <= 1 and (d != 0).mean() < 1e-3
    f32u = torch.empty((9, 1024), dtype=torch.float32, device=DEV)
    ops.pool_blocks(dev_bf16(k), dev_i32(ids), out_f32=f32u, round_bf16=False)
    assert np.array_equal(f32u.cpu().numpy(), G["gsa_krepre"])  # the compiled reference, bit for bit


def test_pool_slots_reps_and_strided_cache(ops, oracle):
    rng = np.random.default_rng(11)
    # K and V interleaved per block ([num_blocks, 2, T, H, D]): block stride is twice the block size,
    # and a cache whose token rows are padded (token stride > H*D)
    kv = H.randn_bf16(rng, (10, 2, 16, 5, 64))
    kvd = dev_bf16(kv)
    k_view = kvd[:, 0, :, :4, :]           # [10, 16, 4, 64], token stride 5*64
    ids = np.array([3, 9, 0, 5], np.int32)
    slots = np.array([6, 1, 4, 2], np.int32)
    table = torch.zeros((8, 4, 3, 64), dtype=torch.bfloat16, device=DEV)
    for r, mode in enumerate(("mean", "max", "min")):
        ops.pool_blocks(k_view, dev_i32(ids), mode=mode, out_slots=dev_i32(slots), out_bf16=table, n_rep=3, rep_index=r)
    got = host_bits(table)
    kk = np.ascontiguousarray(kv[:, 0, :, :4, :])
    for r in range(3):
        want = H.f32_to_bf16(oracle.pool_blocks(kk, ids, r, True)).reshape(4, 4, 64)
        assert np.array_equal(got[slots, :, r, :], want)
    untouched = np.setdiff1d(np.arange(8), slots)
    assert not got[untouched].any()


def test_pool_empty_and_many_blocks(ops, oracle):
    rng = np.random.default_rng(12)
    k = H.randn_bf16(rng, (700, 16, 2, 64))
    kd = dev_bf16(k)
    assert ops.pool_blocks(kd, dev_i32(np.zeros(0))).shape[0] == 0
    ids = rng.integers(0, 700, 1500).astype(np.int32)      # more blocks than resident CTAs, with repeats
    out = ops.pool_blocks(kd, dev_i32(ids))
    want = H.f32_to_bf16(oracle.pool_blocks(k, ids, 0, True))
    assert np.array_equal(host_bits(out).reshape(1500, 128), want)


# ------------------------------------------------------------------------- stage 2 prologue: q

def test_query_group_mean_exact(ops, oracle):
    q = H.case_qmean()
    for rnd in (True, False):
        got = ops.query_group_mean(dev_bf16(q), 8, round_bf16=rnd).cpu().numpy()
        assert np.array_equal(got, oracle.query_group_mean(q, 8, rnd))
    # fewer query heads than KV heads: heads repeat
    q2 = H.randn_bf16(np.random.default_rng(3), (2, 2, 64))
    assert np.array_equal(ops.query_group_mean(dev_bf16(q2), 4).cpu().numpy(), oracle.query_group_mean(q2, 4, True))
    d = H.bf16_ulp_distance(H.f32_to_bf16(ops.query_group_mean(dev_bf16(q), 8).cpu().numpy()), H.f32_to_bf16(G["qmean"]))
    assert d.max() <= 1 and (d != 0).mean() < 1e-3


# ------------------------------------------------------------------------------ stage 2a: dot

def _score_tol(ref):
    scale = float(np.sqrt(np.mean(np.square(ref[np.isfinite(ref)])))) if ref.size else 1.0
    return dict(rtol=1e-3, atol=1e-3 * scale)


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_score_dot_ragged(ops, oracle, dtype):
    rng = np.random.default_rng(21)
    n_slots, E = 900, 1024
    reps16 = H.randn_bf16(rng, (n_slots, E), 0.09)
    reps32 = H.bf16_to_f32(reps16)
    counts = [64, 0, 257, 1, 33, 300, 0, 130]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    slots = rng.integers(0, n_slots, total).astype(np.int32)
    slots[5] = -1
    q = H.bf16_to_f32(H.randn_bf16(rng, (len(counts), E)))
    table = dev_bf16(reps16) if dtype == "bf16" else torch.from_numpy(reps32).to(DEV)
    got = ops.score_dot(table, dev_i32(off), torch.from_numpy(q).to(DEV), total=total, slot_ids=dev_i32(slots),
                        n_kv_heads=8, head_dim=128).cpu().numpy()
    ok = slots >= 0
    ref = oracle.score_dot_esa(reps32, off, np.maximum(slots, 0), q)
    np.testing.assert_allclose(got[ok], ref[ok], **_score_tol(ref))
    assert np.isneginf(got[~ok]).all()
    # identity slots and a scale
    off1 = np.array([0, n_slots], np.int32)
    got1 = ops.score_dot(table, dev_i32(off1), torch.from_numpy(q[:1]).to(DEV), total=n_slots, n_kv_heads=8,
                         head_dim=128, scale=4.0).cpu().numpy()
    ref1 = 4.0 * oracle.score_dot_esa(reps32, off1, None, q[:1])
    np.testing.assert_allclose(got1, ref1, **_score_tol(ref1))


@pytest.mark.parametrize("dtype,Hkv,D", [("bf16", 1, 128), ("bf16", 1, 64), ("bf16", 2, 16), ("f32", 1, 64), ("f32", 2, 16), ("bf16", 1, 16)])
def test_score_dot_narrow_rows(ops, oracle, dtype, Hkv, D):
    """Rows of 32 to 256 bytes (one KV head per rank under head parallelism): several rows per warp, empty requests,
    empty table entries, a range that does not divide by the rows in flight."""
    rng = np.random.default_rng(23)
    n_slots, E = 3001, Hkv * D
    reps16 = H.randn_bf16(rng, (n_slots, E), 0.09)
    reps32 = H.bf16_to_f32(reps16)
    counts = [0, 64, 0, 0, 4099, 1, 33, 3000, 0, 131, 7]
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    slots = rng.integers(0, n_slots, total).astype(np.int32)
    slots[[0, 63, 64, 4000, total - 1]] = -1
    q = H.bf16_to_f32(H.randn_bf16(rng, (len(counts), E)))
    table = dev_bf16(reps16) if dtype == "bf16" else torch.from_numpy(reps32).to(DEV)
    got = ops.score_dot(table, dev_i32(off), torch.from_numpy(q).to(DEV), total=total, slot_ids=dev_i32(slots),
                        n_kv_heads=Hkv, head_dim=D, scale=0.5).cpu().numpy()
    ok = slots >= 0
    ref = 0.5 * oracle.score_dot_esa(reps32, off, np.maximum(slots, 0), q)
    np.testing.assert_allclose(got[ok], ref[ok], **_score_tol(ref))
    assert np.isneginf(got[~ok]).all()
    # identity slots, one request, a total that is not a multiple of anything
    off1 = np.array([0, n_slots], np.int32)
    got1 = ops.score_dot(table, dev_i32(off1), torch.from_numpy(q[1:2]).to(DEV), total=n_slots, n_kv_heads=Hkv,
                         head_dim=D).cpu().numpy()
    ref1 = oracle.score_dot_esa(reps32, off1, None, q[1:2])
    np.testing.assert_allclose(got1, ref1, **_score_tol(ref1))


@pytest.mark.parametrize("Hq,Hkv,D", [(32, 8, 128), (8, 8, 128), (2, 4, 64), (64, 8, 128)])
def test_score_dot_query_fused_equals_two_step(ops, oracle, Hq, Hkv, D):
    """The fused prologue takes the same mean, in the same order, as ucmx_query_group_mean: the scores
    of the one-launch route equal those of the two-launch route bit for bit, and match the checker."""
    rng = np.random.default_rng(23)
    n_slots = 400
    reps16 = H.randn_bf16(rng, (n_slots, Hkv * D), 0.09)
    counts = [130, 0, 77, 1, 192]
    off = H.ragged_offsets(counts)
    slots = rng.integers(0, n_slots, int(off[-1])).astype(np.int32)
    q16 = H.randn_bf16(rng, (len(counts), Hq, D))
    for rnd in (True, False):
        fused = ops.score_dot_query(dev_bf16(reps16), dev_i32(off), dev_bf16(q16), total=int(off[-1]),
                                    slot_ids=dev_i32(slots), n_kv_heads=Hkv, round_bf16=rnd)
        qbar = ops.query_group_mean(dev_bf16(q16), Hkv, round_bf16=rnd)
        two = ops.score_dot(dev_bf16(reps16), dev_i32(off), qbar, total=int(off[-1]), slot_ids=dev_i32(slots),
                            n_kv_heads=Hkv, head_dim=D)
        assert torch.equal(fused, two)
        ref = oracle.score_dot_esa(H.bf16_to_f32(reps16), off, slots, oracle.query_group_mean(q16, Hkv, rnd))
        np.testing.assert_allclose(fused.cpu().numpy(), ref, **_score_tol(ref))


def test_score_dot_matches_compiled_reference(ops):
    data, query, idx, topk = H.case_esa()
    for r in range(3):
        allowed = idx[r][idx[r] >= 0]
        off = np.array([0, len(allowed)], np.int32)
        got = ops.score_dot(torch.from_numpy(data).to(DEV), dev_i32(off), torch.from_numpy(query[r:r + 1]).to(DEV),
                            total=len(allowed), slot_ids=dev_i32(allowed), n_kv_heads=8, head_dim=128).cpu().numpy()
        top = np.sort(got)[::-1][:topk]
        np.testing.assert_allclose(top, G["esa_scores"][r], **_score_tol(G["esa_scores"][r]))


@pytest.mark.parametrize("n_rep,H_,D", [(3, 8, 128), (1, 4, 64), (2, 2, 256), (2, 8, 128), (4, 8, 128), (2, 4, 128), (4, 4, 128),
                                        (2, 1, 128)])
def test_score_dot_gsa_multi_rep(ops, oracle, n_rep, H_, D):
    rng = np.random.default_rng(22)
    n_slots = 120
    reps16 = H.randn_bf16(rng, (n_slots, H_, n_rep, D), 0.09)
    reps32 = H.bf16_to_f32(reps16)
    counts = [50, 70]
    off = H.ragged_offsets(counts)
    slots = rng.permutation(n_slots).astype(np.int32)
    slots[[3, 77]] = -1                      # entries without a block score -inf
    q = H.bf16_to_f32(H.randn_bf16(rng, (2, H_ * D)))
    ok = slots >= 0
    for table in (dev_bf16(reps16), torch.from_numpy(reps32).to(DEV)):
        got = ops.score_dot(table, dev_i32(off), torch.from_numpy(q).to(DEV), total=120, slot_ids=dev_i32(slots),
                            n_kv_heads=H_, head_dim=D, n_rep=n_rep).cpu().numpy()
        ref = oracle.score_dot_gsa(reps32, H_, n_rep, D, off, np.maximum(slots, 0), q)
        np.testing.assert_allclose(got[ok], ref[ok], **_score_tol(ref))
        assert np.isneginf(got[~ok]).all()


def test_score_dot_gsa_reference_vectors(ops):
    for n_rep in (1, 3):
        _, reps, _ = H.case_gsa(n_rep=n_rep)
        qm = torch.from_numpy(G[f"gsa_qmean_r{n_rep}"].reshape(1, -1).copy()).to(DEV)
        got = ops.score_dot(torch.from_numpy(reps).to(DEV), dev_i32([0, 40]), qm, total=40, n_kv_heads=8, head_dim=128,
                            n_rep=n_rep).cpu().numpy()
        np.testing.assert_allclose(got, G[f"gsa_scores_r{n_rep}"], **_score_tol(G[f"gsa_scores_r{n_rep}"]))


# ------------------------------------------------------------------------------ stage 3: top-k

def _ragged_scores(rng, counts, ties):
    off = H.ragged_offsets(counts)
    total = int(off[-1])
    if ties:
        s = rng.integers(-6, 6, total).astype(np.float32) * 0.5   # many equal scores, both zeros
        s[s == 0] = np.where(rng.random((s == 0).sum()) < 0.5, 0.0, -0.0)
    else:
        s = rng.standard_normal(total).astype(np.float32)
    return off, s


@pytest.mark.parametrize("ties", [False, True])
def test_topk_esa_order(ops, oracle, ties):
    rng = np.random.default_rng(31)
    counts = [1, 64, 1000, 0, 5000, 2049, 17]
    off, s = _ragged_scores(rng, counts, ties)
    ks = np.array([1, 16, 50, 4, 2048, 300, 40], np.int32)
    ids = rng.integers(0, 10**6, len(s)).astype(np.int32)
    idx, sc, cnt = ops.topk_ragged(torch.from_numpy(s).to(DEV), dev_i32(off), dev_i32(ks), out_stride=2048,
                                   id_map=dev_i32(ids))
    idx, sc, cnt = idx.cpu().numpy(), sc.cpu().numpy(), cnt.cpu().numpy()
    for r, n in enumerate(counts):
        wi, ws = oracle.topk_esa(s[off[r]:off[r + 1]], int(ks[r]), ids[off[r]:off[r + 1]])
        assert cnt[r] == len(wi) == min(n, ks[r])
        assert np.array_equal(idx[r, :cnt[r]], wi)
        assert np.array_equal(sc[r, :cnt[r]], ws)      # -0.0 == 0.0 compares equal, as in the checker
        assert (idx[r, cnt[r]:] == -1).all()


@pytest.mark.parametrize("ties", [False, True])
def test_topk_gsa_windows(ops, oracle, ties):
    rng = np.random.default_rng(32)
    counts = [256, 5, 6, 7, 40, 1500, 3000, 12]
    off, s = _ragged_scores(rng, counts, ties)
    ks = np.array([64, 3, 6, 7, 6, 200, 0, 20], np.int32)
    idx, _, cnt = ops.topk_ragged(torch.from_numpy(s).to(DEV), dev_i32(off), dev_i32(ks), out_stride=3000, start_win=2,
                                  end_win=4, window_mode=ops.WIN_FORCE, order=ops.ORDER_INDEX_ASC, want_scores=False)
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    for r, n in enumerate(counts):
        want = oracle.topk_gsa(s[off[r]:off[r + 1]], int(ks[r]), 2, 4, cap=3000)
        assert cnt[r] == len(want), (r, cnt[r], len(want))
        assert np.array_equal(idx[r, :cnt[r]], want)


def test_topk_gsa_reference_vectors(ops):
    for n_rep in (1, 3):
        s = torch.from_numpy(G[f"gsa_scores_r{n_rep}"].copy()).to(DEV)
        idx, _, cnt = ops.topk_ragged(s, dev_i32([0, 40]), dev_i32([12]), out_stride=12, start_win=2, end_win=4,
                                      window_mode=ops.WIN_FORCE, order=ops.ORDER_INDEX_ASC, want_scores=False)
        assert cnt.item() == 12 and np.array_equal(idx.cpu().numpy()[0], G[f"gsa_topk_r{n_rep}"])


def test_topk_kvcomp_int_scores(ops, oracle):
    rng = np.random.default_rng(33)
    counts = [7, 300, 3, 2, 1200]
    off = H.ragged_offsets(counts)
    s = rng.integers(-2000, 2000, int(off[-1])).astype(np.int32)
    ks = np.array([3, 30, 5, 1, 120], np.int32)
    idx, sc, cnt = ops.topk_ragged(torch.from_numpy(s).to(DEV), dev_i32(off), dev_i32(ks), out_stride=1200, start_win=1,
                                   end_win=1, window_mode=ops.WIN_EXCLUDE, order=ops.ORDER_INDEX_ASC)
    idx, sc, cnt = idx.cpu().numpy(), sc.cpu().numpy(), cnt.cpu().numpy()
    for r in range(len(counts)):
        seg = s[off[r]:off[r + 1]]
        want = oracle.topk_kvcomp(seg, int(ks[r]), 1, 2)
        assert cnt[r] == len(want)
        assert np.array_equal(idx[r, :cnt[r]], want)
        assert np.array_equal(sc[r, :cnt[r]], seg[want])
    # the reference's own vector
    sg = torch.from_numpy(G["kvcomp_scores_all"].copy()).to(DEV)
    idx, _, cnt = ops.topk_ragged(sg, dev_i32([0, 7]), dev_i32([3]), out_stride=8, start_win=1, end_win=1,
                                  window_mode=ops.WIN_EXCLUDE, order=ops.ORDER_INDEX_ASC, want_scores=False)
    assert np.array_equal(idx.cpu().numpy()[0, :cnt.item()], G["kvcomp_topk"])


# ------------------------------------------------------------------------------ KVComp hashing

def test_hash_encode_bit_exact(ops, oracle):
    w, q, keys = H.case_hash()
    wd = dev_bf16(w)
    assert np.array_equal(ops.hash_encode(dev_bf16(q), wd).cpu().numpy(), oracle.hash_encode(q, w))
    assert np.array_equal(ops.hash_encode(dev_bf16(keys), wd).cpu().numpy(), oracle.hash_encode(keys, w))
    rng = np.random.default_rng(41)
    x = H.randn_bf16(rng, (1000, 128))          # not a multiple of the tile
    got = ops.hash_encode(dev_bf16(x), wd).cpu().numpy()
    assert np.array_equal(got, oracle.hash_encode(x, w))
    # agreement with the reference encoder, up to bits whose projection is within rounding of zero
    ref = G["hash_k_codes"]
    mine = ops.hash_encode(dev_bf16(keys), wd).cpu().numpy()
    assert np.unpackbits(mine ^ ref).mean() < 1e-4


def test_hash_encode_blocks_paged(ops, oracle):
    rng = np.random.default_rng(42)
    w = H.randn_bf16(rng, (128, 256), 2.0)
    k = H.randn_bf16(rng, (9, 16, 4, 128))
    ids = np.array([8, 0, 3, 3, 5], np.int32)
    want = oracle.hash_encode(k[ids], w)                                   # [5, 16, 4, 32]
    got_tm = ops.hash_encode_blocks(dev_bf16(k), dev_i32(ids), dev_bf16(w), head_major=False).cpu().numpy()
    assert np.array_equal(got_tm, want)
    slots = np.array([4, 2, 0, 1, 3], np.int32)
    out = torch.zeros((5, 4, 16, 32), dtype=torch.uint8, device=DEV)
    ops.hash_encode_blocks(dev_bf16(k), dev_i32(ids), dev_bf16(w), out_slots=dev_i32(slots), out=out)
    assert np.array_equal(out.cpu().numpy()[slots], want.transpose(0, 2, 1, 3))


@pytest.mark.parametrize("cross", [True, False])
def test_score_hamming_exact(ops, oracle, cross):
    rng = np.random.default_rng(43)
    n_slots = 300
    codes = rng.integers(0, 256, (n_slots, 8, 128, 16), dtype=np.uint8)
    counts = [70, 0, 129, 31]
    off = H.ragged_offsets(counts)
    slots = rng.integers(0, n_slots, int(off[-1])).astype(np.int32)
    qc = rng.integers(0, 256, (4, 8, 16), dtype=np.uint8)
    got = ops.score_hamming(torch.from_numpy(codes).to(DEV), dev_i32(off), torch.from_numpy(qc).to(DEV),
                            total=int(off[-1]), slot_ids=dev_i32(slots), cross_head=cross).cpu().numpy()
    assert np.array_equal(got, oracle.score_hamming(codes, off, slots, qc, cross))


def test_score_hamming_other_shapes_and_reference(ops, oracle):
    rng = np.random.default_rng(44)
    codes = rng.integers(0, 256, (40, 4, 16, 32), dtype=np.uint8)    # 256-bit codes, 16-token blocks
    qc = rng.integers(0, 256, (2, 4, 32), dtype=np.uint8)
    off = np.array([0, 25, 40], np.int32)
    for cross in (True, False):
        got = ops.score_hamming(torch.from_numpy(codes).to(DEV), dev_i32(off), torch.from_numpy(qc).to(DEV), total=40,
                                cross_head=cross).cpu().numpy()
        assert np.array_equal(got, oracle.score_hamming(codes, off, None, qc, cross))
    kc = np.ascontiguousarray(G["hash_k_codes"].transpose(0, 2, 1, 3))
    got = ops.score_hamming(torch.from_numpy(kc).to(DEV), dev_i32([0, 7]), torch.from_numpy(G["hash_q_codes"]).to(DEV),
                            total=7).cpu().numpy()
    assert np.array_equal(got, G["kvcomp_scores_all"])


# ------------------------------------------------------------------------------ stage 4: blocks

@pytest.mark.parametrize("host", [False, True])
def test_gather_scatter_bit_exact(ops, oracle, host):
    rng = np.random.default_rng(51)
    nb, slice_elems = 96, 16 * 4 * 64            # 8 KiB slices of bf16
    kv = rng.integers(0, 2**16, (2, nb, slice_elems), dtype=np.uint16)
    kvd = torch.from_numpy(kv.view(np.int16)).to(DEV)
    ids = rng.permutation(nb)[:40].astype(np.int32)
    ids[7] = -1
    nbytes = 40 * 2 * slice_elems * 2
    if host:
        staging = torch.zeros(nbytes, dtype=torch.uint8).pin_memory()
    else:
        staging = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)
    ops.gather_blocks([kvd[0], kvd[1]], dev_i32(ids), staging)
    torch.cuda.synchronize()
    planes = [kv[0].view(np.uint8).reshape(nb, -1), kv[1].view(np.uint8).reshape(nb, -1)]
    want = oracle.gather_blocks(planes, np.maximum(ids, 0), slice_elems * 2, slice_elems * 2)
    got = staging.cpu().numpy().reshape(40, 2, -1)
    keep = ids >= 0
    assert np.array_equal(got[keep], want[keep]) and not got[~keep].any()
    # scatter into fresh slots and compare the whole pool
    dst = rng.permutation(nb)[:40].astype(np.int32)
    dst[3] = -1
    pool = torch.zeros_like(kvd)
    ops.scatter_blocks([pool[0], pool[1]], dev_i32(dst), staging)
    torch.cuda.synchronize()
    ref = [np.zeros_like(planes[0]), np.zeros_like(planes[1])]
    ok = dst >= 0
    oracle.scatter_blocks(ref, dst[ok], slice_elems * 2, slice_elems * 2, np.ascontiguousarray(got[ok]))
    out = pool.cpu().numpy().view(np.uint16).view(np.uint8).reshape(2, nb, -1)
    assert np.array_equal(out[0], ref[0]) and np.array_equal(out[1], ref[1])


def test_gather_odd_slice_and_copy_batch(ops):
    rng = np.random.default_rng(52)
    # slice of 16400 bytes: one full 16 KiB chunk plus a 16-byte tail
    pool = torch.from_numpy(rng.integers(0, 255, (20, 16400), dtype=np.uint8)).to(DEV)
    ids = dev_i32([4, 19, 0])
    st = torch.zeros(3 * 16400, dtype=torch.uint8, device=DEV)
    ops.gather_blocks([pool], ids, st)
    assert torch.equal(st.view(3, 16400), pool[ids.long()])
    # pointer-pair form (the IDevice batch call)
    src = torch.from_numpy(rng.integers(0, 255, (5, 4096), dtype=np.uint8)).to(DEV)
    dst = torch.zeros_like(src)
    sp = torch.tensor([src[i].data_ptr() for i in (3, 1, 4)], dtype=torch.int64, device=DEV)
    dp = torch.tensor([dst[i].data_ptr() for i in (0, 2, 4)], dtype=torch.int64, device=DEV)
    ops.copy_batch(dp, sp, 4096)
    torch.cuda.synchronize()
    assert torch.equal(dst[0], src[3]) and torch.equal(dst[2], src[1]) and torch.equal(dst[4], src[4])
    assert not dst[1].any() and not dst[3].any()
    from ucmx import _native
    assert _native.device_error() == 0


# ------------------------------------------------------------- full-size, size-independent checks

def test_full_size_properties(ops):
    """Llama-3-8B KV shapes at the benchmark's scale: properties that need no CPU reference."""
    g = torch.Generator(device=DEV).manual_seed(2002)
    nb = 2048                                                     # 512 MiB of K
    k = torch.randn((nb, 128, 8, 128), generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    ids = torch.randperm(nb, generator=g, device=DEV).to(torch.int32)
    reps = ops.pool_blocks(k, ids)
    # pooling is a permutation-equivariant map: pooling blocks in order then permuting is the same
    base = ops.pool_blocks(k, torch.arange(nb, device=DEV, dtype=torch.int32))
    assert torch.equal(reps, base[ids.long()])
    # mean lies between min and max, element-wise
    mx = ops.pool_blocks(k, ids[:64], mode="max").float()
    mn = ops.pool_blocks(k, ids[:64], mode="min").float()
    assert bool(((reps[:64].float() <= mx) & (reps[:64].float() >= mn)).all())
    # scoring is linear in q: score(2q) == 2 score(q) exactly (power-of-two scale)
    off = torch.tensor([0, 700, nb], dtype=torch.int32, device=DEV)
    q = torch.randn((2, 1024), generator=g, device=DEV)
    s1 = ops.score_dot(reps, off, q, total=nb, slot_ids=ids, n_kv_heads=8, head_dim=128)
    s2 = ops.score_dot(reps, off, 2 * q, total=nb, slot_ids=ids, n_kv_heads=8, head_dim=128)
    assert torch.equal(s2, 2 * s1)
    # top-k: the selected set is exactly the k largest, in order
    kk = torch.tensor([35, 68], dtype=torch.int32, device=DEV)
    idx, sc, cnt = ops.topk_ragged(s1, off, kk, out_stride=68)
    for r, (a, b) in enumerate(((0, 700), (700, nb))):
        ref = torch.sort(s1[a:b], descending=True, stable=True)
        n = int(kk[r])
        assert torch.equal(sc[r, :n], ref.values[:n]) and torch.equal(idx[r, :n].long(), ref.indices[:n])
    # gather then scatter through staging restores every selected block bit for bit
    v = torch.randn((nb, 128, 8, 128), generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    sel = ids[:512].contiguous()
    staging = torch.empty(512 * 2 * 262144, dtype=torch.uint8, device=DEV)
    ops.gather_blocks([k, v], sel, staging)
    k2, v2 = torch.zeros_like(k), torch.zeros_like(v)
    ops.scatter_blocks([k2, v2], sel, staging)
    assert torch.equal(k2[sel.long()], k[sel.long()]) and torch.equal(v2[sel.long()], v[sel.long()])
    assert int(k2.view(torch.int16).ne(0).any(dim=(1, 2, 3)).sum()) == 512


# ---------------------------------------------------------------- GSA device-side weights (per query head)

def test_score_dot_heads_matches_checker_and_reference(ops, oracle):
    reps, q, off, ids, inc, exc = H.case_gsa_heads()
    dev = "cuda:0"
    t = lambda a: torch.from_numpy(a).to(dev)
    bf = lambda u: torch.from_numpy(u.view(np.int16).copy()).to(dev).view(torch.bfloat16)
    got = ops.score_dot_heads(bf(reps), t(off), bf(q), total=int(off[-1]), slot_ids=t(ids), include_mask=t(inc),
                              exclude_mask=t(exc)).cpu().numpy()
    want = oracle.score_dot_gsa_heads(H.bf16_to_f32(reps), off, ids, q, inc, exc)
    fin = np.isfinite(want)
    assert np.array_equal(np.isposinf(got), np.isposinf(want)) and np.array_equal(np.isneginf(got), np.isneginf(want))
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-4, atol=1e-5)
    ref = np.load(os.path.join(os.path.dirname(__file__), "golden", "gsa_heads.npz"))["weights"]   # the reference, in bf16
    assert np.all(np.abs(got[fin] - ref[fin]) <= 8e-3 * np.maximum(np.abs(got[fin]), 0.5))
    # with one representative per block the weights rank blocks like the group-mean dot product does
    one = ops.score_dot_heads(bf(reps[:, :, :1].copy()), t(off), bf(q), total=int(off[-1]), slot_ids=t(ids)).cpu().numpy()
    esa = ops.score_dot_query(bf(reps[:, :, :1].copy()), t(off), bf(q), total=int(off[-1]), slot_ids=t(ids), n_kv_heads=8).cpu().numpy()
    np.testing.assert_allclose(one * 8, esa, rtol=0, atol=0.06)      # esa rounds the group mean of q to bf16 (values ~ +-10)


@pytest.mark.parametrize("Hq,Hkv,R", [(32, 8, 2), (64, 8, 2), (16, 4, 4)])
def test_score_dot_heads_many_short_requests(ops, oracle, Hq, Hkv, R):
    """Requests of one to three candidates: a thread block's candidates then belong to more requests than it keeps
    queries for in shared memory, so both ways of fetching a query are taken inside one launch."""
    rng = np.random.default_rng(Hq + R)
    counts = rng.integers(1, 4, size=90)
    off = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    total = int(off[-1])
    n_slots = total + 7
    reps = H.randn_bf16(rng, (n_slots, Hkv, R, 128), 0.5)
    q = H.randn_bf16(rng, (len(counts), Hq, 128))
    ids = rng.permutation(n_slots)[:total].astype(np.int32)
    ids[[5, total - 2]] = -1
    dev = "cuda:0"
    bf = lambda u: torch.from_numpy(u.view(np.int16).copy()).to(dev).view(torch.bfloat16)
    got = ops.score_dot_heads(bf(reps), torch.from_numpy(off).to(dev), bf(q), total=total, slot_ids=torch.from_numpy(ids).to(dev)).cpu().numpy()
    want = oracle.score_dot_gsa_heads(H.bf16_to_f32(reps), off, ids, q)
    fin = np.isfinite(want)
    assert np.array_equal(np.isneginf(got), np.isneginf(want)) and (~fin).sum() == 2
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("Hq,Hkv,D,R", [(8, 8, 128, 2), (64, 8, 128, 1), (4, 2, 64, 5), (32, 1, 32, 3), (32, 8, 128, 2), (16, 4, 128, 4),
                                        (8, 1, 128, 2), (64, 8, 128, 4), (16, 8, 128, 2)])
def test_score_dot_heads_shapes(ops, oracle, Hq, Hkv, D, R):
    rng = np.random.default_rng(Hq * 131 + R)
    n_slots = 50
    reps = H.randn_bf16(rng, (n_slots, Hkv, R, D), 0.5)
    q = H.randn_bf16(rng, (2, Hq, D))
    off = np.array([0, 19, 50], np.int32)
    ids = rng.permutation(n_slots).astype(np.int32)
    ids[3] = -1
    dev = "cuda:0"
    bf = lambda u: torch.from_numpy(u.view(np.int16).copy()).to(dev).view(torch.bfloat16)
    got = ops.score_dot_heads(bf(reps), torch.from_numpy(off).to(dev), bf(q), total=50, slot_ids=torch.from_numpy(ids).to(dev)).cpu().numpy()
    want = oracle.score_dot_gsa_heads(H.bf16_to_f32(reps), off, ids, q)
    assert np.isneginf(got[3]) and np.isneginf(want[3])
    fin = np.isfinite(want)
    np.testing.assert_allclose(got[fin], want[fin], rtol=1e-4, atol=1e-5)
