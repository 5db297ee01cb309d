"""ucmx.gsa_offload_ops.CalKpreAndTopk driven the way ucm/sparse/gsa/gsa.py drives the reference object, its top-k
cache compared with TopkBlockSelector::SelectTopK of the compiled reference (or the CPU checker's restatement)."""
import time

import numpy as np
import pytest
import torch

import helpers as H

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _expected(oracle, q, reps, Hkv, Hq, D, k):
    """SelectTopK for one request: q [Hq, D] fp32, reps [n, Hkv, 1, D] fp32."""
    n_out = reps.shape[0] if (k >= reps.shape[0] or 3 >= reps.shape[0] or k == 0) else k
    if oracle.have_ref():
        return oracle.ref_gsa_select_topk(q.copy(), reps, Hkv, Hq, 1, D, 1, 2, k)[:n_out]
    qbar = q.reshape(Hkv, Hq // Hkv, D).mean(1).reshape(1, -1).astype(np.float32)
    n = reps.shape[0]
    s = oracle.score_dot_gsa(reps, Hkv, 1, D, np.array([0, n], np.int32), None, qbar)
    return oracle.topk_gsa(s, k, 1, 2)


@pytest.mark.parametrize("cache_on_device", [True, False])
def test_cal_kpre_and_topk_follows_the_reference_object(oracle, cache_on_device):
    from ucmx.gsa_offload_ops import CalKpreAndTopk
    rng = np.random.default_rng(401)
    L, T, max_bs, Hq, Hkv, D = 3, 16, 8, 8, 2, 64
    max_blocks = 200
    n_blocks = [150, 0, 40, 3, 97]                   # request 1 is not decoding, request 3 is shorter than its k
    is_decode = [True, False, True, True, True]
    topk_lens = [45, 12, 3, 30]                      # one per decoding request (request 3: k >= n -> identity)
    n_slots = 600
    tables32 = [H.bf16_to_f32(H.randn_bf16(rng, (n_slots, 1, Hkv, D), 0.3)) for _ in range(L)]
    slot_mapping, pos = [], 0
    for n in n_blocks:
        slot_mapping.append(list(range(pos, pos + n)))          # the reference reads a contiguous range from the first slot
        pos += n
    ops_obj = CalKpreAndTopk(L, T, max_bs, Hq, D, device=torch.device(DEV))
    ops_obj.set_kpre_method_param(Hkv, 1)
    ops_obj.set_kpre_cache([torch.from_numpy(t).to(DEV) for t in tables32])
    assert ops_obj.is_calculate_finish()                          # nothing asked yet: the reference's flags start true
    where = DEV if cache_on_device else "cpu"
    caches = [torch.full((len(n_blocks), max_blocks), -7, dtype=torch.int32, device=where) for _ in range(L)]
    cal_idx = [i for i, d in enumerate(is_decode) if d]
    for rnd in range(2):                                           # two decode steps with new queries
        ops_obj.set_common_param(cal_idx, is_decode)
        ops_obj.set_topk_param(slot_mapping)
        ops_obj.set_topk_cache(caches, topk_lens)
        queries = [H.bf16_to_f32(H.randn_bf16(rng, (len(n_blocks), Hq, D))) for _ in range(L)]
        ids = [(7 if d else -1) for d in is_decode]
        for l in range(L):
            qt = torch.from_numpy(queries[l]).to(DEV).to(torch.bfloat16)      # the engine's dtype; the object widens it
            ops_obj.add_copy_req(False, l, ids, qt)
        deadline = time.time() + 10
        while not ops_obj.is_calculate_finish():
            assert time.time() < deadline
            time.sleep(0.001)
        ops_obj.wait()
        for l in range(L):
            got = caches[l].cpu().numpy()
            assert (got[1] == -7).all()                           # the prefill request's row is untouched
            for j, i in enumerate(cal_idx):
                n, k = n_blocks[i], topk_lens[j]
                reps = tables32[l][slot_mapping[i]].reshape(n, Hkv, 1, D)
                want = _expected(oracle, queries[l][i], reps, Hkv, Hq, D, k)
                n_out = len(want)
                assert n_out == (n if (k >= n or 3 >= n) else k)
                assert np.array_equal(got[i, :n_out], want), (rnd, l, i)
                assert (got[i, n_out:] == -7).all()
