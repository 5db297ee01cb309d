"""The CPU restatement of KVStar's softmax-vote retrieval against what the reference's own kernel
returned (tests/golden/kvstar.npz, recorded from both builds of simd_compute_kernel.cpp)."""
import os

import numpy as np
import pytest

import helpers as H

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "kvstar.npz"))


@pytest.mark.parametrize("name", sorted(H.KVSTAR_CASES))
def test_votes_rank_blocks_like_the_reference(oracle, name):
    q, reps, pruned, k = H.case_kvstar(name)
    votes = oracle.kvstar_scores(q, reps, pruned)
    # every query row casts a total vote of one
    assert abs(float(votes.sum()) / (q.shape[0] * q.shape[1]) - 1.0) < 1e-4
    # the scalar build orders all blocks by vote: the restatement must produce that very ranking
    np.testing.assert_array_equal(oracle.kvstar_topk(votes, len(votes)), G[name + "_rank"])
    # the AVX2 build (polynomial exp, different summation order) selects the same set
    np.testing.assert_array_equal(np.sort(oracle.kvstar_topk(votes, k)), G[name + "_avx2"])


@pytest.mark.parametrize("merge", [2, 4])
def test_block_representations_match_torch_expression(oracle, merge):
    k, ids, pruned = H.case_kvstar_repre(merge=merge)
    got = oracle.kvstar_block_repre(k, ids, pruned, merge)
    np.testing.assert_array_equal(got, G[f"repre_m{merge}"])


def test_half_conversions(oracle):
    rng = np.random.default_rng(3)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, np.inf, -np.inf, 65504.0, 65520.0, 65519.9, 6e-8, 2.98e-8, 2.99e-8], np.float32)])
    lib = oracle.lib()
    import ctypes as C
    lib.orc_f32_to_f16.restype = C.c_uint16
    lib.orc_f32_to_f16.argtypes = [C.c_float]
    lib.orc_f16_to_f32.restype = C.c_float
    lib.orc_f16_to_f32.argtypes = [C.c_uint16]
    want = x.astype(np.float16).view(np.uint16)
    got = np.array([lib.orc_f32_to_f16(float(v)) for v in x], np.uint16)
    np.testing.assert_array_equal(got, want)
    allh = np.arange(0, 65536, 7, dtype=np.uint16)
    back = np.array([lib.orc_f16_to_f32(int(h)) for h in allh], np.float32)
    ref = allh.view(np.float16).astype(np.float32)
    np.testing.assert_array_equal(back.view(np.uint32)[~np.isnan(ref)], ref.view(np.uint32)[~np.isnan(ref)])
