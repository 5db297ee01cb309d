"""The N > 1 host logic on CPU: two gloo ranks.  Each rank holds half of the KV heads, computes its
partial block scores (with the CPU checker standing in for the kernel), all-reduces them through
ucmx.parallel.ScoreAllReduce and must arrive at the full-head scores and at identical selections;
the data-parallel partition must cover every request exactly once with balanced loads."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _worker(rank, world, port, out_dir):
    for p in (ROOT, os.path.join(ROOT, "unified-cache-management_b200"), HERE):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import helpers as H
    from oracle import oracle as orc
    from ucmx.parallel import ScoreAllReduce, head_range, partition_requests
    rng = np.random.default_rng(5005)                       # same data on every rank
    Hkv, D, n_slots = 8, 64, 300
    reps = H.bf16_to_f32(H.randn_bf16(rng, (n_slots, Hkv, D), 0.09))
    counts = [120, 40, 97]
    off = H.ragged_offsets(counts)
    slots = rng.integers(0, n_slots, int(off[-1])).astype(np.int32)
    q = H.bf16_to_f32(H.randn_bf16(rng, (3, Hkv, D)))
    lo, hi = head_range(Hkv, rank, world)
    part = orc.score_dot_esa(np.ascontiguousarray(reps[:, lo:hi].reshape(n_slots, -1)), off, slots,
                             np.ascontiguousarray(q[:, lo:hi].reshape(3, -1)))
    t = torch.from_numpy(part.copy())
    red = ScoreAllReduce()
    red(t)
    full = orc.score_dot_esa(reps.reshape(n_slots, -1), off, slots, q.reshape(3, -1))
    np.testing.assert_allclose(t.numpy(), full, rtol=1e-5, atol=1e-5)
    sel = [orc.topk_esa(t.numpy()[off[r]:off[r + 1]], 7, slots[off[r]:off[r + 1]])[0] for r in range(3)]
    # integer (Hamming) scores reduce exactly
    codes = rng.integers(0, 256, (n_slots, Hkv, 16, 16), dtype=np.uint8)
    qc = rng.integers(0, 256, (3, Hkv, 16), dtype=np.uint8)
    hp = orc.score_hamming(np.ascontiguousarray(codes[:, lo:hi]), off, slots, np.ascontiguousarray(qc[:, lo:hi]), False)
    ht = torch.from_numpy(hp.copy())
    red(ht)
    assert np.array_equal(ht.numpy(), orc.score_hamming(codes, off, slots, qc, False))
    parts = partition_requests([300, 10, 500, 120, 64, 800, 77], world)
    np.save(os.path.join(out_dir, f"sel_{rank}.npy"), np.concatenate(sel))
    np.save(os.path.join(out_dir, f"part_{rank}.npy"), np.asarray(parts[rank]))
    assert red.calls == 2
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_tensor_parallel_scores_and_partition(tmp_path):
    world = 2
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    s0, s1 = np.load(tmp_path / "sel_0.npy"), np.load(tmp_path / "sel_1.npy")
    assert np.array_equal(s0, s1)                             # identical selections on both ranks
    p0, p1 = np.load(tmp_path / "part_0.npy"), np.load(tmp_path / "part_1.npy")
    assert sorted(p0.tolist() + p1.tolist()) == list(range(7))
    loads = [300, 10, 500, 120, 64, 800, 77]
    l0, l1 = sum(loads[i] for i in p0), sum(loads[i] for i in p1)
    assert abs(l0 - l1) <= max(loads) and max(l0, l1) <= 0.6 * sum(loads)


def test_partition_is_deterministic_and_head_ranges():
    sys.path.insert(0, os.path.join(ROOT, "unified-cache-management_b200"))
    from ucmx.parallel import head_range, partition_requests
    a = partition_requests([5, 9, 1, 7, 3, 3], 3)
    assert a == partition_requests([5, 9, 1, 7, 3, 3], 3)
    assert sorted(sum(a, [])) == list(range(6))
    assert [head_range(8, r, 4) for r in range(4)] == [(0, 2), (2, 4), (4, 6), (6, 8)]
    with pytest.raises(ValueError):
        head_range(8, 0, 3)
