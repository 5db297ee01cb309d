"""The CPU checker (oracle/) against vectors produced by the reference itself (tests/golden).

Bit-exact wherever the reference's arithmetic is pinned (integer work, and fp32 work whose order
of operations the compiled reference fixes); a stated tolerance elsewhere."""
import os

import numpy as np
import pytest

import helpers as H

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "golden.npz"))


def test_pool_mean_matches_torch_bf16_mean(oracle):
    k, ids = H.case_pool()
    got = H.f32_to_bf16(oracle.pool_blocks(k, ids, oracle.POOL_MEAN, True)).reshape(9, 8, 128)
    ref = G["pool_mean"]
    # Both round an fp32 mean to bf16; torch sums in a different order, so a value that sits on a
    # rounding boundary may land one bf16 step away.  Everything else must be identical.
    d = H.bf16_ulp_distance(got, ref)
    assert d.max() <= 1
    assert (d != 0).mean() < 1e-3
    # and in fp32 terms: within 1e-3 relative except for those boundary cases
    g32, r32 = H.bf16_to_f32(got), H.bf16_to_f32(ref)
    bad = np.abs(g32 - r32) > 1e-3 * np.abs(r32)
    assert np.array_equal(bad, d != 0)


@pytest.mark.parametrize("name,mode", [("pool_max", 1), ("pool_min", 2)])
def test_pool_max_min_exact(oracle, name, mode):
    k, ids = H.case_pool()
    got = H.f32_to_bf16(oracle.pool_blocks(k, ids, mode, True)).reshape(9, 8, 128)
    assert np.array_equal(got, G[name])


def test_pool_sum_close(oracle):
    k, ids = H.case_pool()
    got = H.f32_to_bf16(oracle.pool_blocks(k, ids, oracle.POOL_SUM, True)).reshape(9, 8, 128)
    assert H.bf16_ulp_distance(got, G["pool_sum"]).max() <= 1


def test_pool_fp32_matches_native_krepre_bit_exact(oracle):
    # KRepreComputer (fp32, token-order accumulation) is reproduced exactly by the unrounded mean
    k, ids = H.case_pool()
    got = oracle.pool_blocks(k, ids, oracle.POOL_MEAN, False)
    assert np.array_equal(got, G["gsa_krepre"])


def test_query_group_mean(oracle):
    q = H.case_qmean()
    got = oracle.query_group_mean(q, 8, True)
    ref = G["qmean"]
    d = H.bf16_ulp_distance(H.f32_to_bf16(got), H.f32_to_bf16(ref))
    assert d.max() <= 1 and (d != 0).mean() < 1e-3


def test_query_group_mean_fp32_matches_gsa_native(oracle):
    qg, _, _ = H.case_gsa(n_rep=1)
    got = oracle.query_group_mean(H.f32_to_bf16(qg)[None], 8, False).reshape(8, 128)
    np.testing.assert_allclose(got, G["gsa_qmean_r1"], rtol=1e-6, atol=1e-7)


def test_esa_scores_and_topk_bit_exact(oracle):
    data, query, idx, topk = H.case_esa()
    for r in range(3):
        allowed = idx[r][idx[r] >= 0]
        off = np.array([0, len(allowed)], np.int32)
        s = oracle.score_dot_esa(data, off, allowed, query[r:r + 1])
        ti, ts = oracle.topk_esa(s, topk, allowed)
        assert np.array_equal(ts, G["esa_scores"][r])          # same fp32 bits as the compiled reference
        assert np.array_equal(ti, G["esa_indices"][r])


@pytest.mark.parametrize("n_rep", [1, 3])
def test_gsa_scores_and_topk(oracle, n_rep):
    qg, reps, p = H.case_gsa(n_rep=n_rep)
    qm = G[f"gsa_qmean_r{n_rep}"].reshape(1, -1)
    off = np.array([0, 40], np.int32)
    s = oracle.score_dot_gsa(reps, 8, n_rep, 128, off, None, qm)
    # the reference's dot is an 8-lane AVX2 tree; the checker sums left to right
    np.testing.assert_allclose(s, G[f"gsa_scores_r{n_rep}"], rtol=1e-5, atol=1e-5)
    sel = oracle.topk_gsa(G[f"gsa_scores_r{n_rep}"], p["k"], p["start"], p["end"])
    assert np.array_equal(sel, G[f"gsa_topk_r{n_rep}"])


def test_gsa_topk_degenerate_cases(oracle):
    s = np.arange(10, dtype=np.float32)
    assert np.array_equal(oracle.topk_gsa(s, 12, 2, 4), np.arange(10))      # k >= n
    assert np.array_equal(oracle.topk_gsa(s, 0, 2, 4), np.arange(10))       # k == 0
    assert np.array_equal(oracle.topk_gsa(s, 5, 6, 4), np.arange(10))       # windows cover all
    assert np.array_equal(oracle.topk_gsa(s, 6, 2, 4), [0, 1, 6, 7, 8, 9])  # no room for the middle
    assert np.array_equal(oracle.topk_gsa(s, 7, 2, 4), [0, 1, 5, 6, 7, 8, 9])


def test_hash_codes_match_reference_encoder(oracle):
    w, q, keys = H.case_hash()
    qc = oracle.hash_encode(q, w)
    kc = oracle.hash_encode(keys, w)
    # The reference projects with a library GEMM (order of additions unspecified); a bit may differ
    # only where the projection is within rounding noise of zero.
    for got, ref, x in ((qc, G["hash_q_codes"], q), (kc, G["hash_k_codes"], keys)):
        diff = np.unpackbits(got ^ ref, axis=-1, bitorder="little").astype(bool)
        if diff.any():
            margin = np.abs(oracle.hash_project(x, w))
            scale = np.abs(H.bf16_to_f32(x)).sum(-1, keepdims=True) * 2.0
            assert (margin[diff] <= 1e-5 * np.broadcast_to(scale, margin.shape)[diff]).all()
        assert diff.mean() < 1e-4


def test_hamming_scores_and_kvcomp_topk_exact(oracle):
    kc = np.ascontiguousarray(G["hash_k_codes"].transpose(0, 2, 1, 3))   # [n, H, T, 16]
    qc = G["hash_q_codes"]
    off = np.array([0, kc.shape[0]], np.int32)
    s = oracle.score_hamming(kc, off, None, qc, cross_head=True)
    assert np.array_equal(s, G["kvcomp_scores_all"])
    assert np.array_equal(oracle.topk_kvcomp(s, 3, 1, 2), G["kvcomp_topk"])
    # matched-head variant is the diagonal of the same sum: check it against a direct evaluation
    sm = oracle.score_hamming(kc, off, None, qc, cross_head=False)
    bits_k = np.unpackbits(kc, axis=-1, bitorder="little").astype(np.int32) * 2 - 1
    bits_q = np.unpackbits(qc, axis=-1, bitorder="little").astype(np.int32) * 2 - 1
    direct = np.einsum("hd,nhsd->n", bits_q[0], bits_k)
    assert np.array_equal(sm, direct)


def test_store_offsets(oracle):
    for rank, tp, layer, is_v, want in G["offset_cases"]:
        assert oracle.store_offset(128, 8 // tp, 128, int(rank), int(tp), 2, int(layer), bool(is_v)) == want


def test_gather_scatter_roundtrip(oracle):
    rng = np.random.default_rng(7)
    kp = rng.integers(0, 255, (10, 4096), dtype=np.uint8)
    vp = rng.integers(0, 255, (10, 4096), dtype=np.uint8)
    ids = np.array([7, 2, 9], np.int32)
    st = oracle.gather_blocks([kp, vp], ids, 4096, 4096)
    assert np.array_equal(st[:, 0], kp[ids]) and np.array_equal(st[:, 1], vp[ids])
    k2, v2 = np.zeros_like(kp), np.zeros_like(vp)
    dst = np.array([1, 5, 3], np.int32)
    oracle.scatter_blocks([k2, v2], dst, 4096, 4096, st)
    assert np.array_equal(k2[dst], kp[ids]) and np.array_equal(v2[dst], vp[ids])


def test_gsa_device_weights_match_reference_expression(oracle):
    """The reference evaluates cal_topk in bf16 (two roundings: the dot products and the mean), the checker in
    fp32: agreement to 8e-3 relative, identical +inf / -inf pattern."""
    reps, q, off, ids, inc, exc = H.case_gsa_heads()
    want = np.load(os.path.join(os.path.dirname(__file__), "golden", "gsa_heads.npz"))["weights"]
    got = oracle.score_dot_gsa_heads(H.bf16_to_f32(reps), off, ids, q, inc, exc)
    assert np.array_equal(np.isposinf(got), np.isposinf(want)) and np.array_equal(np.isneginf(got), np.isneginf(want))
    fin = np.isfinite(want)
    assert np.all(np.abs(got[fin] - want[fin]) <= 8e-3 * np.maximum(np.abs(got[fin]), 0.5))
    assert np.isneginf(got[off[1] - 1])          # flagged both ways: excluded


def _same_rounds(mine, ref):
    assert len(mine) == len(ref)
    for a, b in zip(mine, ref):
        maps = [{int(k): int(v) for k, v in m.items()} for m in b["blocks_map"]]
        assert a["table"] == b["table"]                 # block table, in logical order
        assert a["load_blocks"] == b["load_blocks"]     # blocks taken from the free list, in miss order
        assert a["miss_idx"] == b["miss_idx"]
        assert a["free"] == b["free"]                   # the free list left behind
        assert a["blocks_map"] == maps


@pytest.mark.parametrize("name", list(H.REMAP_SCENARIOS))
def test_remap_matches_recorded_prefetch_engine(oracle, name):
    """Recorded runs of the reference's GSAPrefetchEngineC (kvcache_pre.cpp compiled unmodified): tables, load
    lists, free lists and block maps of every layer after every round, all identical."""
    import json
    with open(os.path.join(os.path.dirname(__file__), "golden", "remap_rounds.json")) as f:
        recorded = {c["name"]: c["rounds"] for c in json.load(f)}
    _same_rounds(H.remap_replay(oracle, H.remap_scenario(name)), recorded[name])


def test_remap_matches_live_prefetch_engine(oracle):
    """Random life cycles against the compiled reference itself, when it has been built here."""
    if not oracle.have_prefetch_ref():
        pytest.skip("the reference prefetch engine is not built")
    rng = np.random.default_rng(7200)
    for it in range(25):
        n_logical = int(rng.integers(4, 80))
        n_owned = int(rng.integers(1, n_logical))
        block_table = [int(x) for x in rng.permutation(3 * n_logical)[:n_logical] + 1]
        owned = sorted(int(x) for x in rng.permutation(n_logical)[:n_owned])
        n_free = int(rng.integers(0, n_owned + 1))
        free_idx = sorted((int(x) for x in rng.permutation(owned)[:n_free]), key=lambda i: block_table[i])
        k = int(rng.integers(1, n_logical + 1))
        L = int(rng.integers(1, 4))
        rounds = [np.stack([np.sort(rng.permutation(n_logical)[:k]) if it % 2 else rng.permutation(n_logical)[:k]
                            for _ in range(L)]).astype(np.int64) for _ in range(int(rng.integers(1, 6)))]
        sc = {"n_layers": L, "block_table": block_table, "owned_idx": owned, "free_idx": free_idx, "rounds": rounds,
              "idx_dtype": "int32" if it % 3 else "int64"}
        ref = oracle.ref_prefetch_rounds(L, block_table, owned, free_idx, rounds, req_id=it, idx_dtype=sc["idx_dtype"])
        _same_rounds(H.remap_replay(oracle, sc), ref)
