"""KVStar softmax-vote retrieval on the GPU against the CPU restatement and the reference's recorded
selections.  Votes are fp32 sums of exponentials of half-precision dot products: the tensor-core
kernel adds the products of a dot in its own order and uses the hardware exp2, so votes are compared
within 5e-4 relative (observed differences are ~1e-5); selected sets must be identical whenever the
k-th and (k+1)-th votes differ by more than that."""
import os

import numpy as np
import pytest
import torch

import helpers as H
from ucmx import _native as N
from ucmx import ops

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "kvstar.npz"))
RTOL = 5e-4


def half(bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.float16).cuda()


def run_single(q, reps, pruned):
    n = reps.shape[0]
    off = torch.tensor([0, n], dtype=torch.int32, device="cuda")
    qoff = torch.tensor([0, q.shape[0]], dtype=torch.int32, device="cuda")
    pr = None if pruned is None else torch.from_numpy(pruned).cuda().unsqueeze(0).contiguous()
    out = ops.kvstar_scores(half(reps), off, half(q), qoff, total=n, max_q_tokens=q.shape[0], pruned_index=pr)
    torch.cuda.synchronize()
    assert N.device_error() == 0
    return out.cpu().numpy()


def kernel_choice(q, reps):
    """0 = CUDA cores, 1 = tensor cores one block per tile, 2 = tensor cores two blocks per instruction."""
    n, M, Hk, dp = reps.shape
    return N.lib.ucmx_kvstar_kernel_choice(n, M, Hk, dp, q.shape[0], q.shape[1])


@pytest.mark.parametrize("name", sorted(H.KVSTAR_CASES))
def test_votes_and_selection_match(oracle, name):
    q, reps, pruned, k = H.case_kvstar(name)
    want = oracle.kvstar_scores(q, reps, pruned)
    got = run_single(q, reps, pruned)
    np.testing.assert_allclose(got, want, rtol=RTOL, atol=1e-6)
    srt = np.sort(want)[::-1]
    assert srt[k - 1] - srt[k] > 4 * RTOL * srt[k - 1], "the seeded case must not sit on a tie"
    off = torch.tensor([0, len(got)], dtype=torch.int32, device="cuda")
    kk = torch.tensor([k], dtype=torch.int32, device="cuda")
    idx, _, cnt = ops.topk_ragged(torch.from_numpy(got).cuda(), off, kk, out_stride=k, order=ops.ORDER_SCORE_DESC)
    sel = idx.cpu().numpy().reshape(-1)[:k]
    assert int(cnt.cpu()[0]) == k
    np.testing.assert_array_equal(np.sort(sel), G[name + "_avx2"])            # the reference's selection
    np.testing.assert_array_equal(np.sort(sel), np.sort(G[name + "_rank"][:k]))


def test_the_seeded_cases_cover_every_kernel():
    """The shape decides the kernel; the seeded cases between them run all three, the benchmark shapes on tensor cores."""
    seen = set()
    for name in sorted(H.KVSTAR_CASES):
        q, reps, _, _ = H.case_kvstar(name)
        seen.add(kernel_choice(q, reps))
    for name in ("llama", "qwen", "short_group"):
        q, reps, _, _ = H.case_kvstar(name)
        assert kernel_choice(q, reps) >= 1
    q, reps, _, _ = H.case_kvstar("odd")
    assert kernel_choice(q, reps) == 0
    assert N.lib.ucmx_kvstar_kernel_choice(1000, 64, 8, 32, 8, 32) == 2        # the benchmark's shape
    assert seen == {0, 1, 2}


def test_ragged_batch_with_slots_and_per_request_channels(oracle):
    """Several requests with different numbers of query tokens and blocks, their representations
    scattered over a shared table, each with its own kept-channel list."""
    rng = np.random.default_rng(77)
    Hq, Hk, D, dp, M = 32, 8, 128, 32, 64
    n_blocks = [5, 64, 1, 33, 17]
    xs = [8, 3, 8, 6, 1]
    n_slots = sum(n_blocks) + 9
    table = H.f32_to_f16_bits(rng.standard_normal((n_slots, M, Hk, dp), dtype=np.float32) * np.float32(0.6))
    slots = rng.permutation(n_slots)[:sum(n_blocks)].astype(np.int32)
    q = H.f32_to_f16_bits(rng.standard_normal((sum(xs), Hq, D), dtype=np.float32))
    pruned = np.stack([np.stack([rng.permutation(D)[:dp] for _ in range(Hk)]) for _ in xs]).astype(np.int64)
    off = np.concatenate([[0], np.cumsum(n_blocks)]).astype(np.int32)
    qoff = np.concatenate([[0], np.cumsum(xs)]).astype(np.int32)
    got = ops.kvstar_scores(half(table), torch.from_numpy(off).cuda(), half(q), torch.from_numpy(qoff).cuda(),
                            total=int(off[-1]), max_q_tokens=8, slot_ids=torch.from_numpy(slots).cuda(),
                            pruned_index=torch.from_numpy(pruned).cuda()).cpu().numpy()
    assert N.device_error() == 0
    for r in range(len(xs)):
        want = oracle.kvstar_scores(q[qoff[r]:qoff[r + 1]], table[slots[off[r]:off[r + 1]]], pruned[r])
        np.testing.assert_allclose(got[off[r]:off[r + 1]], want, rtol=RTOL, atol=1e-6)


def test_many_blocks_votes_sum_to_rows():
    """A size the CPU checker would take minutes for: every query row's votes still add up to one."""
    g = torch.Generator(device="cuda").manual_seed(5)
    Hq, H, D, dp, M, n, x = 32, 8, 128, 32, 64, 3000, 8
    reps = (torch.randn((n, M, H, dp), generator=g, device="cuda") * 0.6).to(torch.float16)
    q = torch.randn((2 * x, Hq, D), generator=g, device="cuda").to(torch.float16)
    pr = torch.stack([torch.stack([torch.randperm(D, generator=g, device="cuda")[:dp] for _ in range(H)]) for _ in range(2)])
    off = torch.tensor([0, 1000, n], dtype=torch.int32, device="cuda")
    qoff = torch.tensor([0, x, 2 * x], dtype=torch.int32, device="cuda")
    out = ops.kvstar_scores(reps, off, q, qoff, total=n, max_q_tokens=x, pruned_index=pr.contiguous())
    torch.cuda.synchronize()
    assert N.device_error() == 0
    assert abs(float(out[:1000].sum()) - x * Hq) < 0.05 and abs(float(out[1000:].sum()) - x * Hq) < 0.05
    assert bool((out > 0).all())


@pytest.mark.parametrize("merge", [2, 4])
def test_block_representations_bit_exact(oracle, merge):
    k, ids, pruned = H.case_kvstar_repre(merge=merge)
    kc = torch.from_numpy(k.view(np.int16).copy()).view(torch.bfloat16).cuda()
    got = ops.kvstar_block_repre(kc, torch.from_numpy(ids).cuda(), merge=merge, pruned_index=torch.from_numpy(pruned).cuda())
    got = got.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(got, oracle.kvstar_block_repre(k, ids, pruned, merge))
    np.testing.assert_array_equal(got, G[f"repre_m{merge}"])
    # all channels kept, scattered into table slots
    slots = torch.tensor([4, 0, 6, 1, 3], dtype=torch.int32, device="cuda")
    table = torch.zeros((7, 128 // merge, 8, 128), dtype=torch.float16, device="cuda")
    ops.kvstar_block_repre(kc, torch.from_numpy(ids).cuda(), merge=merge, out_slots=slots, out=table)
    want = oracle.kvstar_block_repre(k, ids, None, merge)
    got = table[slots.long()].cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(got, want)


def test_kvstar_retrieve_module_interface(oracle):
    """The call sequence of ucm/sparse/kvstar/multistep.py: submit, wait, read the result."""
    from ucmx import kvstar as kvstar_retrieve
    q, reps, pruned, k = H.case_kvstar("llama")
    tq = torch.from_numpy(q.view(np.int16).copy()).view(torch.float16)            # host tensors, as the reference passes
    tr = torch.from_numpy(reps.view(np.int16).copy()).view(torch.float16)
    tid = kvstar_retrieve.AsyncRetrieveByCPU(tq, tr, torch.from_numpy(pruned), k, 7, kvstar_retrieve.CPU)
    assert kvstar_retrieve.Wait(tid) == 0
    res = kvstar_retrieve.GetTaskResult(tid)
    assert res["status"] == "SUCCESS" and len(res["data"]) == k
    np.testing.assert_array_equal(np.sort(res["data"]), G["llama_avx2"])
    # best first, like the reference's scalar build
    np.testing.assert_array_equal(res["data"], G["llama_rank"][:k])
    assert kvstar_retrieve.GetTaskResult(10 ** 9) is None
    tid0 = kvstar_retrieve.AsyncRetrieveByCPU(tq, tr, torch.from_numpy(pruned), 0)
    kvstar_retrieve.Wait(tid0)
    assert kvstar_retrieve.GetTaskResult(tid0)["data"] == []
    with pytest.raises(RuntimeError, match="3D"):
        kvstar_retrieve.AsyncRetrieveByCPU(tq[0], tr, None, k)
    with pytest.raises(RuntimeError, match="inconsistent"):
        kvstar_retrieve.AsyncRetrieveByCPU(tq, tr, torch.from_numpy(pruned[:, :8].copy()), k)
